"""Token sampling on a B200: the interface of leat/sampler.py over the CUDA library.

`Sampling`, `GREEDY` and `sample(logits, options, seed, position, seen=None)` keep the names,
argument meaning and result of leat/sampler.py:11-55: logits (B, V) float32, options (B|1, 5)
float32 rows of Sampling.values(), seed (B|1,) uint32, position an int or (B,) int32, seen (B, V)
bool, result (B, 1) int32 on the device.  All tensors are torch CUDA tensors; the work is done by
libleat_sampler.so through ctypes (leat_b200/_lib.py), on the current CUDA stream, without host
synchronisation.  There is no CPU path.

Extensions beyond the reference (keyword-only): `history` / `history_len` / `penalties` for
repetition and frequency penalties from token counts, `uniform` for an inverse-CDF draw from a
supplied uniform per row, and `sample_full()` which also returns the greedy ids, the cut, the
survivor count and the post-filter probabilities.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from leat_b200 import _lib


@dataclass(frozen=True)
class Sampling:
    """How a sequence picks its tokens (leat/sampler.py:11-25): greedily at temperature 0, else by
    drawing from softmax(logits / temperature) over the tokens top_k, top_p and min_p keep;
    presence_penalty comes off the logits of the tokens it has generated, greedy or not."""

    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    presence_penalty: float = 0.0

    def values(self) -> list[float]:
        # a row of the options sample() takes
        return [self.temperature, self.top_k, self.top_p, self.min_p, self.presence_penalty]


GREEDY = Sampling()


@dataclass
class Sampled:
    """Everything one call computes; `ids` is what sample() returns."""

    ids: torch.Tensor  # (B, 1) int32
    greedy: torch.Tensor | None = None  # (B,) int32: argmax of the penalised logits
    cut: torch.Tensor | None = None  # (B,) float32
    kept: torch.Tensor | None = None  # (B,) int32: survivors, scores >= cut
    probs: torch.Tensor | None = None  # (B, width) float32, likeliest first, 0-padded
    prob_ids: torch.Tensor | None = None  # (B, width) int32, -1-padded
    status: torch.Tensor | None = None  # (1,) int32: _lib.STATUS_* bits


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def device_tensor(x):
    """`x` as a torch tensor without copying: torch tensors as they are, any other framework's device
    buffer through DLPack (`__dlpack__`) or the CUDA array interface (`__cuda_array_interface__`:
    numba, CuPy, a tinygrad buffer wrapped in either), so that leat's own tensors can be handed to
    sample() where it keeps them.  Anything else (lists, NumPy arrays) is left to the caller's
    conversion.  The results are torch tensors, which export both protocols in turn."""
    if x is None or isinstance(x, torch.Tensor):
        return x
    if hasattr(x, "__cuda_array_interface__"):
        return torch.as_tensor(x, device="cuda")
    if hasattr(x, "__dlpack__"):
        return torch.from_dlpack(x)
    return x


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class Sampler:
    """A handle of the library with its device workspace, for calls of up to max_rows x max_vocab
    and top_k up to k_max on the single-pass path.  One per device and thread of use, as leat has
    one engine worker (leat/server.py:263)."""

    def __init__(self, max_rows: int, max_vocab: int, k_max: int = 256, device: torch.device | int | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("leat_b200 needs a CUDA device: the sampler has no CPU path")
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else
                                   (device if isinstance(device, int) else device.index or 0))  # fmt: skip
        self.max_rows, self.max_vocab, self.k_max = max_rows, max_vocab, k_max
        size = _lib.lib.leat_sampler_workspace_bytes(max_rows, max_vocab, k_max)
        if size == 0:
            raise ValueError("max_rows and max_vocab must be positive and 0 < k_max <= 1024")
        with torch.cuda.device(self.device):
            self.workspace = torch.empty(size + 256, dtype=torch.uint8, device=self.device)
            base = (self.workspace.data_ptr() + 255) // 256 * 256
            handle = C.c_void_p()
            _lib.check(_lib.lib.leat_sampler_create(base, size, self.device.index, max_rows, max_vocab,
                                                    k_max, C.byref(handle)), "leat_sampler_create")  # fmt: skip
        self.handle = handle

    def __del__(self):
        handle = getattr(self, "handle", None)
        library = getattr(_lib, "lib", None) if _lib is not None else None  # gone at interpreter exit
        if handle and library is not None:
            library.leat_sampler_destroy(handle)
            self.handle = None

    # ---- launch shape -------------------------------------------------------------------------

    def tune(self, threads: int = 0, slices: int = 0) -> None:
        _lib.check(_lib.lib.leat_sampler_tune(self.handle, threads, slices), "leat_sampler_tune")

    def time_kernels(self, enabled: bool = True) -> None:
        """Measurement aid: the kernels of each call stamp their begin and end (also under graph capture)."""
        _lib.check(_lib.lib.leat_sampler_time_kernels(self.handle, int(enabled)), "leat_sampler_time_kernels")

    KERNELS = ("filter_kernel", "finish_list_kernel", "sample_kernel", "floor_kernel", "shard_finish_kernel", "shard_result_kernel")

    def kernel_times(self) -> dict[str, tuple[float, float]]:
        """Begin and end of each kernel of the last call, milliseconds from the first begin (waits for
        the device); kernels the call did not launch are left out."""
        out = (_lib.C.c_float * 12)()
        _lib.check(_lib.lib.leat_sampler_kernel_times(self.handle, out), "leat_sampler_kernel_times")
        return {name: (float(out[2 * k]), float(out[2 * k + 1])) for k, name in enumerate(self.KERNELS) if out[2 * k] >= 0}

    def tune_filter(self, enabled: bool = True) -> None:
        _lib.check(_lib.lib.leat_sampler_tune_filter(self.handle, int(enabled)), "leat_sampler_tune_filter")

    def plan(self, rows: int, vocab: int, history_cap: int = 0) -> tuple[int, int, int]:
        t, s, b = C.c_int32(), C.c_int32(), C.c_int32()
        _lib.check(_lib.lib.leat_sampler_plan(self.handle, rows, vocab, history_cap, C.byref(t),
                                              C.byref(s), C.byref(b)), "leat_sampler_plan")  # fmt: skip
        return t.value, s.value, b.value

    @property
    def last_launches(self) -> int:
        return _lib.lib.leat_sampler_last_launches(self.handle)

    # ---- argument marshalling -------------------------------------------------------------------

    def _args(self, logits, options, seed, position, seen, history, history_len, penalties, uniform,
              flags, vocab_offset=0, vocab_total=0, softcap: float = 0.0) -> tuple[_lib.SampleArgs, list]:  # fmt: skip
        logits, options, seed, seen = device_tensor(logits), device_tensor(options), device_tensor(seed), device_tensor(seen)
        history, history_len, penalties = device_tensor(history), device_tensor(history_len), device_tensor(penalties)
        uniform = device_tensor(uniform)
        position = position if isinstance(position, int) else device_tensor(position)
        formats = {torch.float32: 0, torch.bfloat16: _lib.FLAG_LOGITS_BF16, torch.float16: _lib.FLAG_LOGITS_F16}
        if logits.dim() != 2 or logits.dtype not in formats or not logits.is_cuda:
            raise ValueError("logits must be a (B, V) float32, bfloat16 or float16 CUDA tensor")
        flags |= formats[logits.dtype]
        if logits.stride(1) != 1:
            logits = logits.contiguous()
        rows, vocab = logits.shape
        dev = logits.device
        keep = [logits]  # tensors that must outlive the launch

        def tensor(x, dtype, width=None, name=""):
            if x is None:
                return None, 0
            if not isinstance(x, torch.Tensor):
                x = torch.as_tensor(x, dtype=dtype)
            x = x.to(device=dev, dtype=dtype)
            x = x.reshape(-1, width) if width else x.reshape(-1)
            x = x.contiguous()
            if x.shape[0] not in (rows, 1):
                raise ValueError(f"{name} must have one row, or one per row of logits")
            keep.append(x)
            return x, x.shape[0]

        options, options_rows = tensor(options, torch.float32, 5, "options")
        seed, seed_rows = tensor(seed, torch.uint32 if hasattr(torch, "uint32") else torch.int32, None, "seed")
        # an int position goes by value (leat's graph variable, leat/sampler.py:41-42): no copy, no tensor
        scalar_position = position if isinstance(position, int) and not isinstance(position, bool) else None
        position, position_rows = tensor(None if scalar_position is not None else position, torch.int32, None, "position")
        penalties, penalties_rows = tensor(penalties, torch.float32, 3, "penalties")
        a = _lib.SampleArgs()
        a.logits, a.rows, a.vocab, a.row_stride = logits.data_ptr(), rows, vocab, logits.stride(0)
        a.options, a.options_rows = _ptr(options), options_rows
        a.seed, a.seed_rows = _ptr(seed), seed_rows
        a.position, a.position_rows = _ptr(position), position_rows
        a.penalties, a.penalties_rows = _ptr(penalties), penalties_rows
        if seen is not None:
            if tuple(seen.shape) != (rows, vocab):
                raise ValueError("seen must be (B, V)")
            seen = seen.to(device=dev)
            seen = seen.view(torch.uint8) if seen.dtype == torch.bool else seen.to(torch.uint8)
            if seen.stride(1) != 1:
                seen = seen.contiguous()
            keep.append(seen)
            a.seen, a.seen_stride = seen.data_ptr(), seen.stride(0)
        if history is not None:
            history = history.to(device=dev, dtype=torch.int32)
            if history.dim() != 2 or history.shape[0] != rows:
                raise ValueError("history must be (B, H)")
            history = history.contiguous()
            keep.append(history)
            a.history, a.history_cap = history.data_ptr(), history.shape[1]
            if history_len is not None:
                history_len = history_len.to(device=dev, dtype=torch.int32).reshape(-1).contiguous()
                if history_len.shape[0] != rows:
                    raise ValueError("history_len must be (B,)")
                keep.append(history_len)
                a.history_len = history_len.data_ptr()
            if history.shape[1] == 0:
                a.history, a.history_cap, a.history_len = None, 0, None
        if uniform is not None:
            uniform = uniform.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
            if uniform.shape[0] != rows:
                raise ValueError("uniform must be (B,)")
            keep.append(uniform)
            a.uniform = uniform.data_ptr()
        a.vocab_offset, a.vocab_total, a.flags = vocab_offset, vocab_total, flags | _lib.FLAG_CLEAR_STATUS
        a.softcap, a.position_scalar = float(softcap), int(scalar_position or 0)
        return a, keep

    # ---- entry points ---------------------------------------------------------------------------

    def sample_full(
        self, logits: torch.Tensor, options, seed=None, position=0, seen=None, *,
        history=None, history_len=None, penalties=None, uniform=None, width: int = 0,
        want_greedy: bool = False, want_cut: bool = False, flags: int = 0, out: torch.Tensor | None = None,
        softcap: float = 0.0,
    ) -> Sampled:  # fmt: skip
        a, keep = self._args(logits, options, seed, position, seen, history, history_len, penalties,
                             uniform, flags, softcap=softcap)  # fmt: skip
        rows, dev = a.rows, keep[0].device
        ids = out if out is not None else torch.empty((rows, 1), dtype=torch.int32, device=dev)
        result = Sampled(ids, status=torch.empty(1, dtype=torch.int32, device=dev))  # cleared by the call (FLAG_CLEAR_STATUS)
        a.out_ids, a.status = ids.data_ptr(), result.status.data_ptr()
        if want_greedy:
            result.greedy = torch.empty(rows, dtype=torch.int32, device=dev)
            a.out_greedy = result.greedy.data_ptr()
        if want_cut or width:
            result.cut = torch.empty(rows, dtype=torch.float32, device=dev)
            result.kept = torch.empty(rows, dtype=torch.int32, device=dev)
            a.out_cut, a.out_kept = result.cut.data_ptr(), result.kept.data_ptr()
        if width:
            result.probs = torch.empty((rows, width), dtype=torch.float32, device=dev)
            result.prob_ids = torch.empty((rows, width), dtype=torch.int32, device=dev)
            a.out_probs, a.out_prob_ids, a.out_width = result.probs.data_ptr(), result.prob_ids.data_ptr(), width
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.leat_sample(self.handle, C.byref(a), _stream()), "leat_sample")
        del keep
        return result

    def sample(self, logits, options, seed=None, position=0, seen=None, **extensions) -> torch.Tensor:
        return self.sample_full(logits, options, seed, position, seen, **extensions).ids

    def argmax(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 2 or x.dtype != torch.float32 or not x.is_cuda:
            raise ValueError("x must be a (B, V) float32 CUDA tensor")
        if x.stride(1) != 1:
            x = x.contiguous()
        out = torch.empty((x.shape[0], 1), dtype=torch.int32, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib.leat_argmax(self.handle, x.data_ptr(), x.shape[0], x.shape[1], x.stride(0),
                                            out.data_ptr(), None, _stream()), "leat_argmax")  # fmt: skip
        return out

    def cutoff(self, scores, top_k, top_p, min_p) -> torch.Tensor:
        if scores.dim() != 2 or scores.dtype != torch.float32 or not scores.is_cuda:
            raise ValueError("scores must be a (B, V) float32 CUDA tensor")
        if scores.stride(1) != 1:
            scores = scores.contiguous()
        rows, dev = scores.shape[0], scores.device
        cols = [torch.as_tensor(o, dtype=torch.float32).to(dev).reshape(-1).expand(rows).contiguous()
                for o in (top_k, top_p, min_p)]  # fmt: skip
        cut = torch.empty((rows, 1), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.leat_cutoff(self.handle, scores.data_ptr(), rows, scores.shape[1],
                                            scores.stride(0), cols[0].data_ptr(), cols[1].data_ptr(),
                                            cols[2].data_ptr(), cut.data_ptr(), None, _stream()),
                       "leat_cutoff")  # fmt: skip
        return cut


_SAMPLERS: dict[tuple[int, int], Sampler] = {}


def default_sampler(rows: int, vocab: int, device: torch.device, k_max: int = 256) -> Sampler:
    """The process-wide sampler of a device, regrown when a call exceeds its capacity (the only
    place device memory is allocated; steady-state calls allocate only their outputs)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), k_max)
    have = _SAMPLERS.get(key)
    if have is None or have.max_rows < rows or have.max_vocab < vocab:
        grow_rows = max(rows, have.max_rows if have else 8)
        grow_vocab = max(vocab, have.max_vocab if have else 1 << 18)
        have = _SAMPLERS[key] = Sampler(grow_rows, grow_vocab, k_max, key[0])
    return have


def sample_static(logits: torch.Tensor, options, seed=None, position=0, seen=None, *, history=None,
                  history_len=None, penalties=None, uniform=None, width: int = 0, want_greedy: bool = False,
                  flags: int = 0, out: torch.Tensor | None = None) -> Sampled:  # fmt: skip
    """sample_full() through the library's allocation-free entry point (leat_sample_static): no
    Sampler, no workspace -- the library keeps its scratch in a fixed array of its own.  For
    callers that cannot allocate device memory where they sample.  Up to 64 rows, 262144 tokens and
    top_k 64; all calls on a device share the scratch, so keep them on one stream.  (This Python
    wrapper still creates its output tensors unless `out` is given; the C entry point itself
    allocates nothing.)"""
    a, keep = Sampler._args(None, logits, options, seed, position, seen, history, history_len, penalties,
                            uniform, flags)  # fmt: skip
    rows, dev = a.rows, keep[0].device
    ids = out if out is not None else torch.empty((rows, 1), dtype=torch.int32, device=dev)
    result = Sampled(ids, status=torch.empty(1, dtype=torch.int32, device=dev))  # cleared by the call (FLAG_CLEAR_STATUS)
    a.out_ids, a.status = ids.data_ptr(), result.status.data_ptr()
    if want_greedy:
        result.greedy = torch.empty(rows, dtype=torch.int32, device=dev)
        a.out_greedy = result.greedy.data_ptr()
    if width:
        result.cut = torch.empty(rows, dtype=torch.float32, device=dev)
        result.kept = torch.empty(rows, dtype=torch.int32, device=dev)
        result.probs = torch.empty((rows, width), dtype=torch.float32, device=dev)
        result.prob_ids = torch.empty((rows, width), dtype=torch.int32, device=dev)
        a.out_cut, a.out_kept = result.cut.data_ptr(), result.kept.data_ptr()
        a.out_probs, a.out_prob_ids, a.out_width = result.probs.data_ptr(), result.prob_ids.data_ptr(), width
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.leat_sample_static(C.byref(a), _stream()), "leat_sample_static")
    del keep
    return result


def sample(logits: torch.Tensor, options: torch.Tensor, seed: torch.Tensor, position, seen=None,
           **extensions) -> torch.Tensor:  # fmt: skip
    """leat/sampler.py:31-55: picks one token per row of `logits` (B, V), as its options say;
    returns (B, 1) int32 on the device.  A row's draw depends only on its logits, its options, its
    seed and its position."""
    logits = device_tensor(logits)  # (any framework's device buffer: DLPack or the CUDA array interface)
    sampler = default_sampler(logits.shape[0], logits.shape[1], logits.device)
    return sampler.sample(logits, options, seed, position, seen, **extensions)
