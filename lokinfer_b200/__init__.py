"""B200-native (sm_100a) implementation of lokinfer's Kokoro iSTFTNet generator path.

`ops`        the reference's `ops.*` surface for this path on the `cuda` device (C-ABI library liblkc.so)
`Generator`  the generator graph (models/kokoro/model.py:735-781) wired from those ops
`Decoder`    the AdainResBlk1d stack that produces the generator's input (models/kokoro/model.py:158-221, 704-717)
`timeshard`  one utterance cut along time across the GPUs of a node (halo + statistics exchange over peer memory)
`arena`      planned activation arena for the fixed op sequence of a forward
`synth`      seeded synthetic weights / inputs (random init; no checkpoint is involved)
`sharding`   utterance sharding across GPUs (one process per GPU, no data-path collective)
"""
import importlib

from . import synth  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # torch-dependent parts load on first use so that importing the package stays cheap.
    if name in ("ops", "sharding", "generator", "decoder", "timeshard", "arena", "_lib", "build"):
        return importlib.import_module(f".{name}", __name__)
    if name == "Generator":
        return importlib.import_module(".generator", __name__).Generator
    if name == "Decoder":
        return importlib.import_module(".decoder", __name__).Decoder
    raise AttributeError(name)
