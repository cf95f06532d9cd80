"""jax.custom_vjp around the XLA FFI handlers of grpo_ffi.cc: the replacement for
MLLM_JAX/train_modules/__init__.py:118-180 inside the reference's jitted train step.

NOT RUN where this repository was developed (JAX is not installed there).  Import it only in an
environment with jax >= 0.4.38 and a built libmllm_grpo_ffi.so.  Under a sharded mesh wrap
`grpo_token_loss` in shard_map (rows over ("dp", "fsdp")), because GSPMD replicates the operands of
an opaque custom call; tag `lse` / `grad_coef` with jax.ad_checkpoint.checkpoint_name if the module is
rematerialised (training2.py:61), otherwise the forward runs twice.
"""
import ctypes
import functools
import os

import jax
import jax.numpy as jnp

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = ctypes.CDLL(os.path.join(_HERE, "libmllm_grpo_ffi.so"))
jax.ffi.register_ffi_target("mllm_grpo_fwd", jax.ffi.pycapsule(_lib.MllmGrpoFwd), platform="CUDA")
jax.ffi.register_ffi_target("mllm_grpo_bwd", jax.ffi.pycapsule(_lib.MllmGrpoBwd), platform="CUDA")


@functools.partial(jax.custom_vjp, nondiff_argnums=(6, 7, 8, 9, 10))
def grpo_token_loss(logits, input_ids, labels, advantages, total_valid_token_count, old_per_token_logps,
                    temperature=1.0, epsilon_low=0.2, epsilon_high=0.3, beta=0.0, softcap=0.0):
    """logits [B, L, V] bf16 -> (loss, per_token_logps [B, L-1], token_entropy [B, L-1])."""
    return _fwd(logits, input_ids, labels, advantages, total_valid_token_count, old_per_token_logps, temperature,
                epsilon_low, epsilon_high, beta, softcap)[0]


def _fwd(logits, input_ids, labels, advantages, nv, old_lp, temperature, epsilon_low, epsilon_high, beta, softcap):
    B, L, _ = logits.shape
    T = L - 1
    ids = input_ids[:, 1:].astype(jnp.int32)                   # :118
    mask = labels[:, 1:].astype(jnp.float32)                   # :120
    has_old = old_lp is not None
    dummy = jnp.zeros((B, T), jnp.float32)
    f32 = lambda *s: jax.ShapeDtypeStruct(s, jnp.float32)       # noqa: E731
    loss, lp, ent, lse, gcoef, _terms = jax.ffi.ffi_call(
        "mllm_grpo_fwd", (f32(1), f32(B, T), f32(B, T), f32(B * T), f32(B * T), f32(B * T)))(
        logits, ids, mask, advantages.astype(jnp.float32), old_lp if has_old else dummy, dummy,
        jnp.asarray(nv, jnp.float32).reshape(1), temperature=float(temperature), epsilon_low=float(epsilon_low),
        epsilon_high=float(epsilon_high), beta=float(beta), softcap=float(softcap), scored_rows=T, has_old=has_old,
        has_ref=False)
    out = (loss[0], jax.lax.stop_gradient(lp), jax.lax.stop_gradient(ent))
    return out, (logits, ids, lse, gcoef, jnp.asarray(nv, jnp.float32).reshape(1))


def _bwd(temperature, epsilon_low, epsilon_high, beta, softcap, res, cot):
    logits, ids, lse, gcoef, nv = res
    dlogits = jax.ffi.ffi_call("mllm_grpo_bwd", jax.ShapeDtypeStruct(logits.shape, logits.dtype),
                               input_output_aliases={0: 0})(
        logits, ids, lse, gcoef, nv, jnp.asarray(cot[0], jnp.float32).reshape(1), temperature=float(temperature),
        softcap=float(softcap), scored_rows=logits.shape[1] - 1)
    return dlogits, None, None, None, None, None


grpo_token_loss.defvjp(_fwd, _bwd)
