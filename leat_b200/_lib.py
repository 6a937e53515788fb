"""ctypes binding of libleat_sampler.so (include/leat_sampler.h).  There is no other path: if the
library is missing, importing this module raises."""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# the in-tree build, unless LEAT_SAMPLER_LIBRARY names another build of the same sources
LIBRARY = Path(os.environ.get("LEAT_SAMPLER_LIBRARY") or Path(__file__).resolve().parent / "csrc" / "libleat_sampler.so")

OK, E_ARGUMENT, E_CAPACITY, E_WORKSPACE, E_CUDA, E_DEVICE = 0, -1, -2, -3, -4, -5
STATUS_FALLBACK, STATUS_TRUNCATED, STATUS_INTERNAL, STATUS_PEER = 1, 2, 4, 8
FLAG_DIVIDE, FLAG_NO_FALLBACK, FLAG_LOGITS_BF16, FLAG_LOGITS_F16, FLAG_CLEAR_STATUS = 1, 2, 4, 8, 16

_ERRORS = {
    E_ARGUMENT: "bad argument (null pointer, shape or broadcast row count)",
    E_CAPACITY: "rows, vocabulary or history beyond the handle's capacity",
    E_WORKSPACE: "workspace too small or misaligned",
    E_CUDA: "CUDA runtime error",
    E_DEVICE: "handle belongs to another device",
}

EXPORTS = [
    "leat_sampler_workspace_bytes", "leat_sampler_create", "leat_sampler_destroy",
    "leat_sampler_tune", "leat_sampler_tune_filter", "leat_sampler_plan", "leat_sampler_last_launches",
    "leat_sampler_time_kernels", "leat_sampler_kernel_times",
    "leat_sampler_last_cuda_error", "leat_sample", "leat_argmax", "leat_cutoff",
    "leat_verify_draft", "leat_settle_draft", "leat_topk_local", "leat_sample_from_candidates", "leat_sample_static",
    "leat_candidate_record_bytes", "leat_candidate_record_layout", "leat_sample_from_records",
    "leat_shard_region_bytes", "leat_peer_alloc", "leat_peer_open", "leat_peer_close", "leat_peer_free",
    "leat_shard_create", "leat_shard_destroy", "leat_shard_select", "leat_shard_finish", "leat_shard_result",
]  # fmt: skip


class SampleArgs(C.Structure):
    """struct leat_sample_args"""

    _fields_ = [
        ("logits", C.c_void_p), ("rows", C.c_int32), ("vocab", C.c_int32), ("row_stride", C.c_int64),
        ("options", C.c_void_p), ("options_rows", C.c_int32),
        ("seed", C.c_void_p), ("seed_rows", C.c_int32),
        ("position", C.c_void_p), ("position_rows", C.c_int32),
        ("seen", C.c_void_p), ("seen_stride", C.c_int64),
        ("history", C.c_void_p), ("history_len", C.c_void_p), ("history_cap", C.c_int32),
        ("penalties", C.c_void_p), ("penalties_rows", C.c_int32),
        ("uniform", C.c_void_p),
        ("vocab_offset", C.c_int32), ("vocab_total", C.c_int32), ("flags", C.c_uint32),
        ("out_ids", C.c_void_p), ("out_greedy", C.c_void_p), ("out_cut", C.c_void_p),
        ("out_kept", C.c_void_p), ("out_probs", C.c_void_p), ("out_prob_ids", C.c_void_p),
        ("out_width", C.c_int32), ("status", C.c_void_p),
        ("softcap", C.c_float), ("position_scalar", C.c_int32),
    ]  # fmt: skip


class SamplerError(RuntimeError):
    pass


def _load() -> C.CDLL:
    if not LIBRARY.exists():
        raise ImportError(
            f"{LIBRARY} is missing: build it with `python -m leat_b200.build` (nvcc, sm_100a). "
            "The sampler has no CPU or eager fallback."
        )
    lib = C.CDLL(str(LIBRARY))
    p, i32, i64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
    lib.leat_sampler_workspace_bytes.restype = sz
    lib.leat_sampler_workspace_bytes.argtypes = [i32, i32, i32]
    lib.leat_sampler_create.argtypes = [p, sz, i32, i32, i32, i32, C.POINTER(p)]
    lib.leat_sampler_destroy.argtypes = [p]
    lib.leat_sampler_tune.argtypes = [p, i32, i32]
    lib.leat_sampler_tune_filter.argtypes = [p, i32]
    lib.leat_sampler_plan.argtypes = [p, i32, i32, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]
    lib.leat_sampler_last_launches.argtypes = [p]
    lib.leat_sampler_time_kernels.argtypes = [p, i32]
    lib.leat_sampler_kernel_times.argtypes = [p, C.POINTER(C.c_float)]
    lib.leat_sampler_last_cuda_error.restype = C.c_char_p
    lib.leat_sampler_last_cuda_error.argtypes = []
    lib.leat_sample.argtypes = [p, C.POINTER(SampleArgs), p]
    lib.leat_sample_static.argtypes = [C.POINTER(SampleArgs), p]
    lib.leat_argmax.argtypes = [p, p, i32, i32, i64, p, p, p]
    lib.leat_cutoff.argtypes = [p, p, i32, i32, i64, p, p, p, p, p, p]
    lib.leat_verify_draft.argtypes = [p, p, p, i32, i32, p, p, p]
    lib.leat_settle_draft.argtypes = [p, p, p, p, p, i32, i32, p, p, i32, p, i32, p, p, p]
    lib.leat_topk_local.argtypes = [p, C.POINTER(SampleArgs), p, p, p, p, i32, p]
    lib.leat_sample_from_candidates.argtypes = [p, C.POINTER(SampleArgs), p, p, p, p, i32, i32, p]
    lib.leat_candidate_record_bytes.restype = sz
    lib.leat_candidate_record_bytes.argtypes = [i32, i32]
    lib.leat_candidate_record_layout.argtypes = [i32, i32, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]
    lib.leat_sample_from_records.argtypes = [p, C.POINTER(SampleArgs), p, i32, i32, p]
    lib.leat_shard_region_bytes.restype = sz
    lib.leat_shard_region_bytes.argtypes = [i32, i32, i32]
    lib.leat_peer_alloc.argtypes = [sz, C.POINTER(p), C.c_char_p]
    lib.leat_peer_open.argtypes = [C.c_char_p, C.POINTER(p)]
    lib.leat_peer_close.argtypes = [p]
    lib.leat_peer_free.argtypes = [p]
    lib.leat_shard_create.argtypes = [p, i32, i32, i32, i32, C.POINTER(p), C.POINTER(p)]
    lib.leat_shard_destroy.argtypes = [p]
    lib.leat_shard_select.argtypes = [p, C.POINTER(SampleArgs), p]
    lib.leat_shard_finish.argtypes = [p, C.POINTER(SampleArgs), p]
    lib.leat_shard_result.argtypes = [p, C.POINTER(SampleArgs), p]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if name not in ("leat_sampler_workspace_bytes", "leat_sampler_last_cuda_error", "leat_candidate_record_bytes",
                        "leat_shard_region_bytes"):
            fn.restype = C.c_int
    return lib


lib = _load()


def check(code: int, what: str) -> None:
    if code == OK:
        return
    detail = _ERRORS.get(code, f"error {code}")
    if code == E_CUDA:
        detail += ": " + (lib.leat_sampler_last_cuda_error() or b"").decode()
    error = ValueError if code in (E_ARGUMENT, E_CAPACITY) else SamplerError
    raise error(f"{what}: {detail}")
