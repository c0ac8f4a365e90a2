"""The Kokoro iSTFTNet generator wired from `ops.*_cuda`: the `cuda`-device twin of the generator part of the
reference graph builder (models/kokoro/model.py:735-781) with its building blocks adain_resblock1_fused (:235-247),
adain_resblock1 (:250-260) and the style bank (:67-81, 135-144). The graph structure is the reference's; only the
kernel-name suffix differs.

Generator(sd) uploads a state dict once (weights become device constants, the ConvTranspose weights are packed once,
the AdaIN `fc` layers are concatenated into one style-bank GEMV). forward() runs one utterance on torch's current
stream. capture(t) records the fused graph for one input length into a CUDA graph with static input/output
buffers, so a replay costs one launch.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops
from .synth import shapes

DILATIONS = (1, 3, 5)
RES_KERNELS = (3, 7, 11)


class _NullCtx:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


class Generator:
    def __init__(self, sd: dict, device="cuda"):
        self.device = torch.device(device)
        self.w = {k: ops.to_cuda(np.ascontiguousarray(v, dtype=np.float32), self.device) for k, v in sd.items()}
        for k in list(self.w):
            if ".alpha" in k:  # Snake alpha (1, C, 1) -> (C,)   (model.py:_flat_alpha)
                self.w[k] = self.w[k].reshape(-1).contiguous()
        # Style bank: every `<name>.fc` as one [128, total] weight + bias, names sorted (model.py:67-81).
        names = sorted(k[: -len(".weight")] for k in self.w if k.endswith(".fc.weight"))
        self.bank_wt = torch.cat([self.w[n + ".weight"].t() for n in names], dim=1).contiguous()
        self.bank_b = torch.cat([self.w[n + ".bias"] for n in names]).contiguous()
        self.bank_off, o = {}, 0
        for n in names:
            self.bank_off[n] = (o, self.w[n + ".bias"].shape[0])
            o += self.bank_off[n][1]
        # Polyphase packs of the two upsamplers (model.py:788-793), run once on constants.
        self.ups_wp = None
        if "ups.0.weight" in self.w:  # a state dict of resblocks only is enough for adain_resblock1*
            self.ups_wp = [ops.convt_poly_weights_cuda(self.w["ups.0.weight"], 10, 5),
                           ops.convt_poly_weights_cuda(self.w["ups.1.weight"], 6, 3)]
            self.ups_state = [ops.conv_transpose1d_prepare_f32_cuda(self.w["ups.0.weight"], 10, 5),
                              ops.conv_transpose1d_prepare_f32_cuda(self.w["ups.1.weight"], 6, 3)]
        self.ident128 = torch.stack([torch.zeros(128), torch.ones(128), torch.zeros(128)]).to(self.device).contiguous()
        # Prepared state of every fused-conv weight the tensor-core kernel accepts (packed once, at init).
        self.conv_state = {}
        for k in self.w:
            if k.endswith(".weight") and (".convs1." in k or ".convs2." in k or k == "conv_post.weight"):
                st = ops.conv1d_prepare_f32_cuda(self.w[k])
                if st is not None:
                    self.conv_state[k[: -len(".weight")]] = st
        # The two noise convs (22 -> 256, k 12, stride 6, padding 3; 22 -> 128, k 1) as stride-1 convs over the
        # polyphase view of `har` (ops.space_to_depth_f32_cuda), channels padded to a multiple of 16: the shape the
        # tensor-core conv takes. Packed once, like every other weight.
        self.noise_tc = {}
        for i, (stride, pad) in enumerate(((6, 3), (1, 0))):
            key = f"noise_convs.{i}"
            if key + ".weight" not in sd:
                continue
            wn = np.ascontiguousarray(sd[key + ".weight"], dtype=np.float32)
            rows = -(-wn.shape[1] * stride // 16) * 16
            wp = ops.to_cuda(ops.polyphase_conv_weights(wn, stride, rows), self.device)
            state = ops.conv1d_prepare_f32_cuda(wp)
            if state is not None:
                ident = torch.stack([torch.zeros(rows), torch.ones(rows), torch.zeros(rows)]).to(self.device).contiguous()
                self.noise_tc[i] = (wp, state, ident, stride, pad, wn.shape[2] // stride, rows)
        self._graphs = {}
        self._streams = None

    # ------------------------------------------------------------------ building blocks

    def _noise_conv(self, har, i, keep):
        """noise_convs[i](har) -> (xs, chunk statistics of xs or None); temporaries go to `keep`. On the tensor cores when the polyphase pack
        exists (and the conv path is not "simt"): space-to-depth of har, then a stride-1 conv with an identity
        affine, whose epilogue also gives the statistics the following resblock needs."""
        w = self.w
        if i in self.noise_tc and ops._conv_path != "simt":
            wp, state, ident, stride, pad, taps, rows = self.noise_tc[i]
            y = ops.space_to_depth_f32_cuda(har, stride, pad, taps, rows)
            keep.append(y)
            return ops.conv1d_affine_f32_cuda(y, wp, w[f"noise_convs.{i}.bias"], ident, state=state)
        if i == 0:
            return ops.conv1d_f32_cuda(har, w["noise_convs.0.weight"], w["noise_convs.0.bias"], stride=6, padding=3), None
        return ops.conv1d_f32_cuda(har, w["noise_convs.1.weight"], w["noise_convs.1.bias"]), None

    def style(self, s):
        """fc(style) of every AdaIN as views into one style-bank GEMV (model.py:135-144): name -> f32[2C]."""
        bank = ops.gemm_bias_f32_cuda(s.reshape(1, -1), self.bank_wt, self.bank_b).reshape(-1)
        return lambda name: bank[self.bank_off[name][0]: self.bank_off[name][0] + self.bank_off[name][1]]

    def _snake_conv(self, x, af, alpha_key, conv, k, d, residual=None):
        w = self.w
        return ops.conv1d_snake_f32_cuda(x, w[conv + ".weight"], w[conv + ".bias"], af, w[alpha_key],
                                         residual=residual, padding=d * (k - 1) // 2, dilation=d,
                                         state=self.conv_state.get(conv))

    def adain_resblock1_fused(self, x, gb, prefix, k, x_stats=None):
        n = x.shape[1]
        st = ops.channel_stats_f32_cuda(x) if x_stats is None else x_stats
        for j, d in enumerate(DILATIONS):
            af = ops.adain_affine_f32_cuda(st, gb(f"{prefix}.adain1.{j}.fc"), length=n)
            xt, st1 = self._snake_conv(x, af, f"{prefix}.alpha1.{j}", f"{prefix}.convs1.{j}", k, d)
            af = ops.adain_affine_f32_cuda(st1, gb(f"{prefix}.adain2.{j}.fc"), length=n)
            x, st = self._snake_conv(xt, af, f"{prefix}.alpha2.{j}", f"{prefix}.convs2.{j}", k, 1, residual=x)
        return x, st

    def adain_resblock1(self, x, gb, prefix, k):
        w = self.w
        for j, d in enumerate(DILATIONS):
            xt = ops.adain1d_f32_cuda(x, gb(f"{prefix}.adain1.{j}.fc"))
            xt = ops.snake_f32_cuda(xt, w[f"{prefix}.alpha1.{j}"])
            xt = ops.conv1d_f32_cuda(xt, w[f"{prefix}.convs1.{j}.weight"], w[f"{prefix}.convs1.{j}.bias"],
                                     padding=d * (k - 1) // 2, dilation=d)
            xt = ops.adain1d_f32_cuda(xt, gb(f"{prefix}.adain2.{j}.fc"))
            xt = ops.snake_f32_cuda(xt, w[f"{prefix}.alpha2.{j}"])
            xt = ops.conv1d_f32_cuda(xt, w[f"{prefix}.convs2.{j}.weight"], w[f"{prefix}.convs2.{j}.bias"],
                                     padding=(k - 1) // 2)
            x = ops.add_f32_cuda(xt, x)
        return x

    # ------------------------------------------------------------------ the graph

    def har_from_f0(self, f0, noise):
        """The generator's `har` input from the F0 curve, as the reference graph computes it before the generator
        (models/kokoro/model.py:720-726): harmonic source (9 harmonics, x300, Linear 9 -> 1, tanh) then STFT(n_fft 20,
        hop 5) -> cat(magnitude, phase). f0 f32[T] (one value per frame of x); noise = f32[300 T, 9] (the normal draw
        as an operand) or an int seed (drawn in the kernel, models/kokoro/model.py:721-722) -> f32[22, 60 T + 1]."""
        ops.check("m_source.l_linear.weight" in self.w, "the state dict has no m_source.l_linear weights")
        w9 = self.w["m_source.l_linear.weight"].reshape(9)
        bias = self.w["m_source.l_linear.bias"].reshape(1)
        if isinstance(noise, int):  # a seed: the noise is drawn in the kernel (the variant the reference graph ships)
            src = ops.harmonic_source_rng_f32_cuda(f0, w9, bias, noise)
        else:
            src = ops.harmonic_source_f32_cuda(f0, noise, w9, bias)
        return ops.stft_magphase_f32_cuda(src, n_fft=20, hop=5)

    def forward(self, x, har, s, fused=True, outputs=("audio",), concurrent=True, pad_rows=True):
        """x f32[512, T], har f32[22, 60 T + 1], s f32[128] (cuda tensors) -> the named outputs
        ("audio" f32[300 T], "post" f32[22, 60 T + 1]; with pad_rows the 2-D outputs are [:, :L] views of buffers
        whose rows are padded to a multiple of 4 floats).

        The op sequence is the reference's (model.py:735-781). With concurrent=True (fused graph only) the branches
        that do not depend on each other are queued on side streams, forked from and joined back to torch's current
        stream: the two noise branches (they only need `har`) and, per stage, the three resblocks (they share their
        input). The results are the same; independent persistent conv kernels then fill the SMs that the tail of
        another one leaves idle (a stage-0 conv of the 26 s case has 164 tiles for 148 SMs)."""
        w = self.w
        ops.check(x.dim() == 2 and x.shape[0] == 512, "x must be f32[512, T]")
        sh = shapes(int(x.shape[1]))
        ops.check(tuple(har.shape) == (22, sh["L1"]), f"har must be f32[22, {sh['L1']}]")
        if fused and pad_rows and not ops._pad_rows and ops._conv_path != "simt":
            # the generator owns every intermediate: rows padded to 16 bytes, so that the tensor-core kernels move
            # them with the TMA unit (values do not depend on the pitch)
            with ops.padded_rows():
                return self.forward(x, har, s, fused, outputs, concurrent, pad_rows)
        gb = self.style(s)
        cur = torch.cuda.current_stream(self.device)
        par = fused and concurrent
        side = self._side_streams() if par else None

        def on(stream):
            return torch.cuda.stream(stream) if par else _NullCtx()

        keep = []  # every intermediate stays referenced until all streams are joined
        st = {}
        rb = None
        noise = [None, None]
        if par:
            for i in (0, 1):
                ops.join(side[i], cur)
        for i, (_, _, k_noise) in enumerate(((20, 10, 7), (12, 6, 11))):
            if not fused:
                break
            with on(side[i] if par else None):
                xs, xs_stats = self._noise_conv(har, i, keep)
                noise[i], _ = self.adain_resblock1_fused(xs, gb, f"noise_res.{i}", k_noise, x_stats=xs_stats)
                keep += [xs, xs_stats] if xs_stats is not None else [xs]
        for i, (k_up, u, k_noise) in enumerate(((20, 10, 7), (12, 6, 11))):
            if fused:
                if par:
                    ops.join(cur, side[i])
                if i == 0:
                    xin = x
                else:
                    # resblock mean as its own pass (13 us of HBM time at T = 2080), so that the upsampler takes the
                    # tensor-core path; conv_transpose1d_poly(..., mean3=...) is the fused CUDA-core alternative
                    xin = ops.add3_scale_f32_cuda(rb[0], rb[1], rb[2], scale=1.0 / 3.0)
                    keep.append(xin)
                x = ops.conv_transpose1d_poly_f32_cuda(
                    xin, self.ups_wp[i], w[f"ups.{i}.bias"], noise[i], stride=u, padding=(k_up - u) // 2,
                    taps=k_up // u, slope=0.1, pad_left=1 if i == 1 else 0, state=self.ups_state[i])
                xst = ops.channel_stats_f32_cuda(x)
                keep += [x, xst, *(rb or [])]
                new_rb = [None, None, None]
                if par:
                    ops.join(side[2], cur)
                    ops.join(side[3], cur)
                # the k = 11 block is the longest: it stays on the current stream
                for j, stream in ((2, None), (1, side[2] if par else None), (0, side[3] if par else None)):
                    with on(stream):
                        new_rb[j] = self.adain_resblock1_fused(x, gb, f"resblocks.{3 * i + j}", RES_KERNELS[j], xst)[0]
                if par:
                    ops.join(cur, side[2])
                    ops.join(cur, side[3])
                rb = new_rb
            else:
                if i == 0:
                    xs = ops.conv1d_f32_cuda(har, w["noise_convs.0.weight"], w["noise_convs.0.bias"], stride=6, padding=3)
                else:
                    xs = ops.conv1d_f32_cuda(har, w["noise_convs.1.weight"], w["noise_convs.1.bias"])
                xs = self.adain_resblock1(xs, gb, f"noise_res.{i}", k_noise)
                x = ops.leaky_relu_f32_cuda(x, slope=0.1)
                x = ops.conv_transpose1d_f32_cuda(x, w[f"ups.{i}.weight"], w[f"ups.{i}.bias"], stride=u,
                                                  padding=(k_up - u) // 2, output_padding=0)
                if i == 1:
                    x = ops.pad_reflect1d_f32_cuda(x, left=1, right=0)
                x = ops.add_f32_cuda(x, xs)
                rb = [self.adain_resblock1(x, gb, f"resblocks.{3 * i + j}", kk) for j, kk in enumerate(RES_KERNELS)]
                x = ops.add3_scale_f32_cuda(rb[0], rb[1], rb[2], scale=1.0 / 3.0)
            st[f"stage{i}"] = rb if fused else x
        if fused:
            # resblock mean, then the direct fused conv (model.py:774-776): on this device the extra pass over the
            # mean costs ~40 us of HBM time, and the conv then runs on the tensor cores (Co = 22 padded to 128 rows)
            xm = ops.add3_scale_f32_cuda(rb[0], rb[1], rb[2], scale=1.0 / 3.0)
            post, _ = ops.conv1d_leaky_f32_cuda(xm, w["conv_post.weight"], w["conv_post.bias"], self.ident128,
                                                slope=0.01, padding=3, state=self.conv_state.get("conv_post"))
        else:
            x = ops.leaky_relu_f32_cuda(x, slope=0.01)
            post = ops.conv1d_f32_cuda(x, w["conv_post.weight"], w["conv_post.bias"], padding=3)
        st["post"] = post
        st["audio"] = ops.istft_logits_f32_cuda(post, n_fft=20, hop=5)
        if par:
            # tensors made on a side stream are consumed on the current one: tell the allocator
            for t in keep + noise + list(rb):
                if isinstance(t, torch.Tensor):
                    t.record_stream(cur)
        res = tuple(st[o] for o in outputs)
        return res[0] if len(res) == 1 else res

    def _side_streams(self):
        if self._streams is None:
            self._streams = [torch.cuda.Stream(device=self.device) for _ in range(4)]
        return self._streams

    def _warm_stream(self):
        """The stream capture() runs its warm-up and traced forwards on: one per generator, and never the same CUDA
        stream as a side stream. torch hands streams out of a pool of 32 round-robin, so a stream made later can BE an
        earlier one; a traced forward whose main stream coincided with a side stream would look more serial than the
        captured one is, and the memory plan made from it would overlay tensors of branches that run concurrently."""
        if getattr(self, "_warm", None) is None:
            taken = {s.cuda_stream for s in self._side_streams()}
            for _ in range(64):
                s = torch.cuda.Stream(device=self.device)
                if s.cuda_stream not in taken:
                    self._warm = s
                    break
            else:
                raise RuntimeError("no CUDA stream distinct from the side streams")
        return self._warm

    # ------------------------------------------------------------------ CUDA graph replay

    def capture(self, t: int, planned: bool = True):
        """Records forward(fused=True) for input length t into a CUDA graph (once per t). Returns a dict with the
        static buffers `x`, `har`, `s`, `audio` and the `graph`; fill the inputs, then graph.replay().

        planned=True (default): the forward's intermediates live in a planned arena (arena.py): one traced forward
        gives every tensor's life, the plan overlays tensors that are never alive together (judged by the fork / join
        structure of the streams, not by program order), and the captured forward takes views of ONE device buffer
        sized by the plan (`arena_bytes`; `unplanned_bytes` is what keeping every intermediate would take)."""
        if t in self._graphs:
            return self._graphs[t]
        from .arena import PlannedArena, Tracer
        sh = shapes(t)
        dev = self.device
        pitch = -(-t // ops.ROW_ALIGN) * ops.ROW_ALIGN  # rows of x start on 16-byte boundaries for any t
        bufs = {"x": torch.zeros(512, pitch, device=dev)[:, :t], "har": torch.zeros(22, sh["L1"], device=dev),
                "s": torch.zeros(128, device=dev)}
        side = self._warm_stream()
        side.wait_stream(torch.cuda.current_stream(dev))
        arena = None
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up outside capture: lazy module loading, function attributes
                ref = self.forward(bufs["x"], bufs["har"], bufs["s"])
            if planned:
                with ops.tracing(Tracer()) as tr:
                    tr.pin(self.forward(bufs["x"], bufs["har"], bufs["s"]))
                arena = PlannedArena(tr, dev)
                del tr
                arena.begin()
                with ops.use_allocator(arena.allocator):
                    again = self.forward(bufs["x"], bufs["har"], bufs["s"])
                torch.cuda.synchronize(dev)
                ops.check(torch.equal(again, ref), "the planned arena changed the result of the forward")
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            if arena is not None:
                arena.begin()
                with ops.use_allocator(arena.allocator):
                    bufs["audio"] = self.forward(bufs["x"], bufs["har"], bufs["s"])
            else:
                bufs["audio"] = self.forward(bufs["x"], bufs["har"], bufs["s"])
        bufs["graph"] = g
        if arena is not None:
            bufs["arena"], bufs["arena_bytes"], bufs["unplanned_bytes"] = arena, arena.nbytes, arena.unplanned_bytes
        self._graphs[t] = bufs
        return bufs

    def synthesize_f0(self, x_host, f0_host, seed, s_host, audio_host=None):
        """End-to-end call with HOST buffers that starts one step earlier than synthesize(): the `har` input is
        computed on the device from the F0 curve f32[T] (harmonic source with in-kernel noise from `seed`, then the
        STFT), as the reference graph does before its generator (models/kokoro/model.py:720-726)."""
        t = int(x_host.shape[1])
        b = self.capture(t)
        f0 = torch.empty(t, dtype=torch.float32, device=self.device)
        f0.copy_(f0_host, non_blocking=True)
        b["x"].copy_(x_host, non_blocking=True)
        b["s"].copy_(s_host, non_blocking=True)
        b["har"].copy_(self.har_from_f0(f0, int(seed)))
        b["graph"].replay()
        if audio_host is None:
            audio_host = torch.empty(b["audio"].shape, dtype=torch.float32, pin_memory=True)
        audio_host.copy_(b["audio"], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        status = ops.conv_tc_status()
        if status != 0:
            raise RuntimeError(f"tensor-core conv kernels reported status {status:#x}")
        return audio_host

    def pipeline(self, t: int, depth: int = 2):
        """Host-buffer synthesis with `depth` utterances of `t` frames in flight (see SynthesisPipeline)."""
        return SynthesisPipeline(self, t, depth)

    def synthesize(self, x_host, har_host, s_host, audio_host=None):
        """End-to-end call with HOST buffers (pinned torch tensors for async copies): host -> device copies, one
        graph replay, device -> host copy of the waveform. Returns the host waveform tensor. Raises if the tensor-core
        kernels reported a problem during the call (a bounded wait that gave up, or an activation beyond the f16
        range of the split operands, which overflows there and makes the waveform wrong)."""
        t = int(x_host.shape[1])
        b = self.capture(t)
        b["x"].copy_(x_host, non_blocking=True)
        b["har"].copy_(har_host, non_blocking=True)
        b["s"].copy_(s_host, non_blocking=True)
        b["graph"].replay()
        if audio_host is None:
            audio_host = torch.empty(b["audio"].shape, dtype=torch.float32, pin_memory=True)
        audio_host.copy_(b["audio"], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        status = ops.conv_tc_status()
        if status != 0:
            raise RuntimeError(f"tensor-core conv kernels reported status {status:#x} "
                               "(0x10000 = activation beyond the f16 range; else role << 8 | wait that gave up)")
        return audio_host


class SynthesisPipeline:
    """Throughput form of Generator.synthesize for a stream of utterances of one length: the host -> device copies of
    utterance i + 1 and the device -> host copy of utterance i - 1 run on the two copy engines while the captured graph
    computes utterance i. One graph and one arena; per slot a set of staging tensors (inputs and waveform), so the
    graph's static buffers are only touched by device-side copies on the compute stream.

        pipe = gen.pipeline(t)
        tickets = [pipe.submit(x, har, s, out) for (x, har, s, out) in batch]   # pinned host tensors
        for k in tickets: pipe.wait(k)                                          # out is complete after wait

    submit() blocks only when all `depth` slots are in flight (it then waits for the oldest). wait() raises if the
    tensor-core kernels reported a problem up to and including that utterance (the status word is read stream-ordered
    after each utterance, not cleared)."""

    def __init__(self, gen, t: int, depth: int = 2):
        ops.check(depth >= 1, "depth must be >= 1")
        self.gen, self.t, self.depth = gen, int(t), int(depth)
        dev = gen.device
        self.b = gen.capture(self.t)
        self.h2d, self.d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.compute = torch.cuda.current_stream(dev)  # the graph replays on the stream current at construction
        self.slots = []
        for _ in range(self.depth):
            self.slots.append({
                "x": torch.empty_like(self.b["x"]), "har": torch.empty_like(self.b["har"]),
                "s": torch.empty_like(self.b["s"]), "audio": torch.empty_like(self.b["audio"]),
                "status": torch.zeros(1, dtype=torch.int32).pin_memory(),
                "in_ready": torch.cuda.Event(), "in_free": None, "computed": torch.cuda.Event(),
                "out_done": None, "ticket": -1})
        self.n = 0

    def submit(self, x_host, har_host, s_host, audio_host):
        slot = self.slots[self.n % self.depth]
        if slot["ticket"] >= 0:
            self.wait(slot["ticket"])  # the slot's previous utterance has left the device
        b = self.b
        with torch.cuda.stream(self.h2d):
            if slot["in_free"] is not None:
                self.h2d.wait_event(slot["in_free"])
            slot["x"].copy_(x_host, non_blocking=True)
            slot["har"].copy_(har_host, non_blocking=True)
            slot["s"].copy_(s_host, non_blocking=True)
            slot["in_ready"].record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(slot["in_ready"])
            b["x"].copy_(slot["x"]), b["har"].copy_(slot["har"]), b["s"].copy_(slot["s"])
            slot["in_free"] = torch.cuda.Event()
            slot["in_free"].record(self.compute)
            b["graph"].replay()
            slot["audio"].copy_(b["audio"])
            ops.conv_tc_status_async(slot["status"])
            slot["computed"].record(self.compute)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(slot["computed"])
            audio_host.copy_(slot["audio"], non_blocking=True)
            slot["out_done"] = torch.cuda.Event()
            slot["out_done"].record(self.d2h)
        slot["ticket"] = self.n
        self.n += 1
        return slot["ticket"]

    def wait(self, ticket: int) -> None:
        slot = self.slots[ticket % self.depth]
        if slot["ticket"] != ticket:
            return  # already waited for (its slot has been reused or released)
        slot["out_done"].synchronize()
        slot["ticket"] = -1
        status = int(slot["status"].item())
        if status != 0:
            raise RuntimeError(f"tensor-core conv kernels reported status {status:#x} "
                               "(0x10000 = activation beyond the f16 range; else role << 8 | wait that gave up)")
