"""leat_b200: a B200-native token sampler behind the interface of leat/sampler.py.

The work is done by libleat_sampler.so (CUDA, sm_100a), built in-tree by
`python -m leat_b200.build`.  Names are resolved on first use; touching any of them without the
library raises ImportError: there is no CPU or eager fallback."""

_LAZY = {
    "Sampling": "sampler", "GREEDY": "sampler", "sample": "sampler", "Sampler": "sampler",
    "Sampled": "sampler", "default_sampler": "sampler", "ops": None, "speculative": None,
    "sharded": None, "workloads": None, "history": None, "SlotHistory": "history",
}  # fmt: skip


def __getattr__(name):
    import importlib

    if name not in _LAZY:
        raise AttributeError(name)
    module = importlib.import_module(f"leat_b200.{_LAZY[name] or name}")
    return module if _LAZY[name] is None else getattr(module, name)
