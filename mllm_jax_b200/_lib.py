"""ctypes binding of `libmllm_grpo.so` (the C ABI declared in include/mllm_grpo.h).

There is no CPU fallback: if the library is missing or fails to load, every
operator raises.  Loading does not need a GPU; launching does.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libmllm_grpo.so"

FLAG_SKIP_ENTROPY = 1
FLAG_CE_LOSS = 2
LM_HEAD_FLAG_WEIGHT_HV = 256
DEV_ID_CLAMPED = 1
DEV_WAIT_TIMEOUT = 2

EXPORTS = (
    "mllm_grpo_fwd", "mllm_grpo_bwd", "mllm_grpo_fwd_bwd", "mllm_grpo_fwd_partials", "mllm_grpo_combine",
    "mllm_grpo_logprobs", "mllm_grpo_workspace_bytes", "mllm_grpo_abi_version", "mllm_grpo_status_string",
    "mllm_grpo_last_cuda_error", "mllm_grpo_launch_count", "mllm_grpo_fwd_static_scratch",
    "mllm_grpo_fwd_bwd_sharded", "mllm_grpo_exchange_bytes", "mllm_grpo_set_plan_override",
    "mllm_grpo_entropy_stats", "mllm_grpo_scale_grad", "mllm_ppo_value_loss", "mllm_ppo_value_workspace_bytes",
    "mllm_lm_head_partials", "mllm_lm_head_splits", "mllm_lm_head_partials_bytes", "mllm_grpo_partial_width",
)


class GrpoArgs(C.Structure):
    """Mirror of `struct mllm_grpo_args`; field order and types must match the header."""

    _fields_ = [
        ("struct_size", C.c_uint64),
        ("n_seqs", C.c_int64), ("seq_rows", C.c_int64), ("scored_rows", C.c_int64), ("vocab", C.c_int64),
        ("row_stride", C.c_int64), ("vocab_start", C.c_int64), ("vocab_total", C.c_int64),
        ("temperature", C.c_float), ("epsilon_low", C.c_float), ("epsilon_high", C.c_float), ("beta", C.c_float),
        ("softcap", C.c_float), ("adv_per_token", C.c_int32), ("flags", C.c_int32), ("grad_scale", C.c_float),
        ("total_valid", C.c_float),
        ("logits", C.c_void_p), ("chosen_ids", C.c_void_p), ("mask", C.c_void_p), ("advantages", C.c_void_p),
        ("old_logps", C.c_void_p), ("ref_logps", C.c_void_p), ("total_valid_dev", C.c_void_p),
        ("grad_scale_dev", C.c_void_p),
        ("per_token_logps", C.c_void_p), ("token_entropy", C.c_void_p), ("lse", C.c_void_p),
        ("grad_coef", C.c_void_p), ("loss", C.c_void_p), ("loss_terms", C.c_void_p),
        ("dlogits", C.c_void_p),
        ("partials", C.c_void_p), ("gathered_partials", C.c_void_p), ("n_shards", C.c_int32),
        ("shard_rank", C.c_int32),
        ("device_status", C.c_void_p),
        ("peer_exchange", C.c_void_p * 8), ("exchange_epoch", C.c_int32), ("peer_wait_ms", C.c_int32),
        ("sample_entropy", C.c_void_p), ("sample_entropy_window", C.c_void_p),
        ("entropy_cotangent", C.c_void_p), ("lse_scaled", C.c_void_p),
    ]


class PpoValueArgs(C.Structure):
    """Mirror of `struct mllm_ppo_value_args`."""

    _fields_ = [
        ("struct_size", C.c_uint64),
        ("n_seqs", C.c_int64), ("seq_rows", C.c_int64), ("scored_rows", C.c_int64),
        ("clip_range", C.c_float), ("grad_scale", C.c_float), ("total_valid", C.c_float), ("adv_per_token", C.c_int32),
        ("total_valid_dev", C.c_void_p),
        ("values", C.c_void_p), ("returns", C.c_void_p), ("advantages", C.c_void_p), ("old_values", C.c_void_p),
        ("mask", C.c_void_p), ("dvalues", C.c_void_p), ("out", C.c_void_p), ("workspace", C.c_void_p),
    ]


class LmHeadArgs(C.Structure):
    """Mirror of `struct mllm_lm_head_args`."""

    _fields_ = [
        ("struct_size", C.c_uint64),
        ("n_rows", C.c_int64), ("vocab", C.c_int64), ("hidden_dim", C.c_int64), ("hidden_stride", C.c_int64),
        ("weight_stride", C.c_int64), ("vocab_start", C.c_int64), ("vocab_total", C.c_int64),
        ("softcap", C.c_float), ("flags", C.c_int32),
        ("hidden", C.c_void_p), ("weight", C.c_void_p), ("chosen_ids", C.c_void_p), ("partials", C.c_void_p),
        ("device_status", C.c_void_p),
    ]


class GrpoError(RuntimeError):
    def __init__(self, fn: str, status: int, text: str, cuda: str = ""):
        self.status = status
        super().__init__(f"{fn} failed: status {status} ({text})" + (f": {cuda}" if cuda else ""))


_lib = None


def load():
    """Load the library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mllm_jax_b200.build` (needs nvcc). "
            "There is no CPU fallback for the GRPO loss kernels."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name in ("mllm_grpo_fwd", "mllm_grpo_bwd", "mllm_grpo_fwd_bwd", "mllm_grpo_fwd_partials",
                 "mllm_grpo_combine", "mllm_grpo_logprobs", "mllm_grpo_fwd_static_scratch",
                 "mllm_grpo_fwd_bwd_sharded", "mllm_grpo_entropy_stats",
                 "mllm_grpo_scale_grad"):
        fn = getattr(lib, name)
        fn.argtypes = [C.POINTER(GrpoArgs), C.c_void_p]
        fn.restype = C.c_int
    lib.mllm_ppo_value_loss.argtypes = [C.POINTER(PpoValueArgs), C.c_void_p]
    lib.mllm_ppo_value_loss.restype = C.c_int
    lib.mllm_grpo_partial_width.argtypes = [C.POINTER(GrpoArgs)]
    lib.mllm_grpo_partial_width.restype = C.c_int32
    lib.mllm_lm_head_partials.argtypes = [C.POINTER(LmHeadArgs), C.c_void_p]
    lib.mllm_lm_head_partials.restype = C.c_int
    lib.mllm_lm_head_splits.argtypes = [C.c_int64, C.c_int64]
    lib.mllm_lm_head_splits.restype = C.c_int32
    lib.mllm_lm_head_partials_bytes.argtypes = [C.c_int64, C.c_int64]
    lib.mllm_lm_head_partials_bytes.restype = C.c_int64
    lib.mllm_ppo_value_workspace_bytes.argtypes = [C.c_int64, C.c_int64]
    lib.mllm_ppo_value_workspace_bytes.restype = C.c_int64
    lib.mllm_grpo_workspace_bytes.argtypes = [C.c_int64]
    lib.mllm_grpo_workspace_bytes.restype = C.c_int64
    lib.mllm_grpo_set_plan_override.argtypes = [C.c_int] * 5
    lib.mllm_grpo_set_plan_override.restype = C.c_int
    lib.mllm_grpo_exchange_bytes.argtypes = [C.c_int64, C.c_int32]
    lib.mllm_grpo_exchange_bytes.restype = C.c_int64
    lib.mllm_grpo_abi_version.restype = C.c_int
    lib.mllm_grpo_status_string.argtypes = [C.c_int]
    lib.mllm_grpo_status_string.restype = C.c_char_p
    lib.mllm_grpo_last_cuda_error.restype = C.c_char_p
    lib.mllm_grpo_launch_count.restype = C.c_int64
    _lib = lib
    return lib


def call(name: str, args, stream: int) -> None:
    """Invoke one launcher; raise GrpoError on a non-zero status."""
    lib = load()
    args.struct_size = C.sizeof(type(args))
    status = getattr(lib, name)(C.byref(args), C.c_void_p(stream))
    if status != 0:
        raise GrpoError(name, status, lib.mllm_grpo_status_string(status).decode(),
                        lib.mllm_grpo_last_cuda_error().decode())


def launch_count() -> int:
    return int(load().mllm_grpo_launch_count())


class plan_override:
    """Context manager over mllm_grpo_set_plan_override (tuning and tests): forces the separate sweeps,
    or the cluster size / thread count / load batch / shared-memory staging of the one-kernel path, for the
    calls made inside the block; the automatic plan is restored on exit."""

    def __init__(self, sweeps: bool = False, cluster: int = 0, threads: int = 0, load_batch: int = 0,
                 staged: int = -1):
        self.values = (int(bool(sweeps)), int(cluster), int(threads), int(load_batch), int(staged))

    def __enter__(self):
        load().mllm_grpo_set_plan_override(*self.values)
        return self

    def __exit__(self, *exc):
        load().mllm_grpo_set_plan_override(0, 0, 0, 0, -1)
        return False
