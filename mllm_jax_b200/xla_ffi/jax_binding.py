"""jax.custom_vjp around the XLA FFI handlers of grpo_ffi.cc: the replacement for
MLLM_JAX/train_modules/__init__.py:118-180 inside the reference's jitted train step.

EXPERIMENTAL, NOT RUN where this repository was developed: JAX is installed neither there nor on the GPU
hosts it was measured on (`import jax` fails on both), so this module has never been imported.  Use it only
in an environment with jax >= 0.4.38 and a built libmllm_grpo_ffi.so.

What a maintainer wires up:
  * `grpo_token_loss(...)`: loss, per_token_logps, token_entropy with a custom_vjp.  eager=True (default)
    takes the one-kernel path the benchmarks quote: the forward calls mllm_grpo_fwd_bwd (loss and dlogits,
    logits read from HBM once) and the backward only applies the cotangent (a no-op kernel when it is 1, as
    under jax.value_and_grad of the loss, plugins/training/update/train_step.py:24).  eager=False is the
    two-sweep form (mllm_grpo_fwd / mllm_grpo_bwd) whose residuals are two [B*T] vectors.
  * `token_logprobs(...)`: forward-only log-probs (reference model; first PPO epoch, update/ppo.py:39-43).
  * `per_sample_entropy(...)`: the 'entropy' / 'entropy_loss' monitors (:141-157).
  * `sharded_grpo_token_loss(mesh, ...)`: the same under the reference's mesh.  GSPMD replicates the operands
    of an opaque custom call, so the call sits inside shard_map with rows over ("dp", "fsdp"); every shard's
    loss is already divided by the GLOBAL total_valid_token_count (runner/grpo_gsm8k.py:770), so one psum of
    a scalar finishes it.
  * Residuals carry jax.ad_checkpoint.checkpoint_name("grpo_loss_residuals") so the remat wrapper of
    training2.py:61 can be given a policy that keeps them instead of running the forward twice.
Float attributes are passed as numpy float32 / int64 scalars: the handlers decode f32 and i64, and a Python
float would arrive as f64.
"""
import ctypes
import functools
import os

import jax
import jax.numpy as jnp
import numpy as np
from jax.ad_checkpoint import checkpoint_name

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = ctypes.CDLL(os.path.join(_HERE, "libmllm_grpo_ffi.so"))
for _name, _sym in (("mllm_grpo_fwd", "MllmGrpoFwd"), ("mllm_grpo_bwd", "MllmGrpoBwd"),
                    ("mllm_grpo_fwd_bwd", "MllmGrpoFwdBwd"), ("mllm_grpo_scale_grad", "MllmGrpoScaleGrad"),
                    ("mllm_grpo_logprobs", "MllmGrpoLogprobs"), ("mllm_grpo_entropy_stats", "MllmGrpoEntropyStats")):
    jax.ffi.register_ffi_target(_name, jax.ffi.pycapsule(getattr(_lib, _sym)), platform="CUDA")


def _f32(*shape):
    return jax.ShapeDtypeStruct(shape, jnp.float32)


def _attrs(temperature, epsilon_low, epsilon_high, beta, softcap, scored_rows, has_old, has_ref):
    return dict(temperature=np.float32(temperature), epsilon_low=np.float32(epsilon_low),
                epsilon_high=np.float32(epsilon_high), beta=np.float32(beta), softcap=np.float32(softcap or 0.0),
                scored_rows=np.int64(scored_rows), has_old=bool(has_old), has_ref=bool(has_ref))


@functools.partial(jax.custom_vjp, nondiff_argnums=(7, 8, 9, 10, 11, 12))
def grpo_token_loss(logits, input_ids, labels, advantages, total_valid_token_count, old_per_token_logps,
                    ref_per_token_logps, temperature=1.0, epsilon_low=0.2, epsilon_high=0.3, beta=0.0, softcap=0.0,
                    eager=True):
    """logits [B, L, V] bf16 -> (loss, per_token_logps [B, L-1], token_entropy [B, L-1]).
    old_per_token_logps / ref_per_token_logps may be None (ratio == 1 / no KL term)."""
    return _fwd(logits, input_ids, labels, advantages, total_valid_token_count, old_per_token_logps,
                ref_per_token_logps, temperature, epsilon_low, epsilon_high, beta, softcap, eager)[0]


def _fwd(logits, input_ids, labels, advantages, nv, old_lp, ref_lp, temperature, epsilon_low, epsilon_high, beta,
         softcap, eager):
    B, L, _ = logits.shape
    T = L - 1
    ids = input_ids[:, 1:].astype(jnp.int32)                   # :118
    mask = labels[:, 1:].astype(jnp.float32)                   # :120
    has_old, has_ref = old_lp is not None, ref_lp is not None
    dummy = jnp.zeros((B, T), jnp.float32)
    nv = jnp.asarray(nv, jnp.float32).reshape(1)
    operands = (logits, ids, mask, advantages.astype(jnp.float32), old_lp if has_old else dummy,
                ref_lp if has_ref else dummy, nv)
    attrs = _attrs(temperature, epsilon_low, epsilon_high, beta, softcap, T, has_old, has_ref)
    small = (_f32(1), _f32(B, T), _f32(B, T), _f32(B * T), _f32(B * T), _f32(B * T))
    if eager:
        loss, lp, ent, _lse, _gcoef, _terms, dlogits = jax.ffi.ffi_call(
            "mllm_grpo_fwd_bwd", small + (jax.ShapeDtypeStruct(logits.shape, logits.dtype),))(*operands, **attrs)
        res = (checkpoint_name(dlogits, "grpo_loss_residuals"),)
    else:
        loss, lp, ent, lse, gcoef, _terms = jax.ffi.ffi_call("mllm_grpo_fwd", small)(*operands, **attrs)
        res = (logits, ids, checkpoint_name(lse, "grpo_loss_residuals"),
               checkpoint_name(gcoef, "grpo_loss_residuals"), nv)
    out = (loss[0], jax.lax.stop_gradient(lp), jax.lax.stop_gradient(ent))
    return out, res


def _bwd(temperature, epsilon_low, epsilon_high, beta, softcap, eager, res, cot):
    g = jnp.asarray(cot[0], jnp.float32).reshape(1)
    if eager:
        (dlogits,) = res
        dlogits = jax.ffi.ffi_call("mllm_grpo_scale_grad", jax.ShapeDtypeStruct(dlogits.shape, dlogits.dtype),
                                   input_output_aliases={0: 0})(dlogits, g)
    else:
        logits, ids, lse, gcoef, nv = res
        dlogits = jax.ffi.ffi_call("mllm_grpo_bwd", jax.ShapeDtypeStruct(logits.shape, logits.dtype),
                                   input_output_aliases={0: 0})(
            logits, ids, lse, gcoef, nv, g, temperature=np.float32(temperature), softcap=np.float32(softcap or 0.0),
            scored_rows=np.int64(logits.shape[1] - 1))
    return dlogits, None, None, None, None, None, None


grpo_token_loss.defvjp(_fwd, _bwd)


def token_logprobs(logits, input_ids, temperature=1.0, softcap=0.0):
    """Forward-only per_token_logps / token_entropy / lse [B, L-1] (no gradient)."""
    B, L, _ = logits.shape
    T = L - 1
    lp, ent, lse = jax.ffi.ffi_call("mllm_grpo_logprobs", (_f32(B, T), _f32(B, T), _f32(B, T)))(
        jax.lax.stop_gradient(logits), input_ids[:, 1:].astype(jnp.int32), temperature=np.float32(temperature),
        softcap=np.float32(softcap or 0.0), scored_rows=np.int64(T))
    return lp, ent, lse


def per_sample_entropy(token_entropy, labels):
    """'entropy' and 'entropy_loss' [B] of the reference's return dict (train_modules/__init__.py:141-157)."""
    B = token_entropy.shape[0]
    return jax.ffi.ffi_call("mllm_grpo_entropy_stats", (_f32(B), _f32(B)))(
        token_entropy, labels[:, 1:].astype(jnp.float32))


def sharded_grpo_token_loss(mesh, logits, input_ids, labels, advantages, total_valid_token_count,
                            old_per_token_logps=None, ref_per_token_logps=None, **attrs):
    """grpo_token_loss with the batch split over the mesh axes ("dp", "fsdp") (tp = 1, every configuration the
    reference ships): each device runs the kernel on its own rows, the scalar losses are summed."""
    from jax.experimental.shard_map import shard_map
    from jax.sharding import PartitionSpec as P

    rows = ("dp", "fsdp")
    B, L, _ = logits.shape
    has_old, has_ref = old_per_token_logps is not None, ref_per_token_logps is not None
    dummy = jnp.zeros((B, L - 1), jnp.float32)

    def local(lg, ids, lab, adv, nv, old, ref):
        loss, lp, ent = grpo_token_loss(lg, ids, lab, adv, nv, old if has_old else None, ref if has_ref else None,
                                        attrs.get("temperature", 1.0), attrs.get("epsilon_low", 0.2),
                                        attrs.get("epsilon_high", 0.3), attrs.get("beta", 0.0),
                                        attrs.get("softcap", 0.0), attrs.get("eager", True))
        return jax.lax.psum(loss, rows), lp, ent

    return shard_map(local, mesh=mesh,
                     in_specs=(P(rows, None, None), P(rows, None), P(rows, None), P(rows), P(), P(rows, None),
                               P(rows, None)),
                     out_specs=(P(), P(rows, None), P(rows, None)), check_rep=False)(
        logits, input_ids, labels, advantages, jnp.asarray(total_valid_token_count, jnp.float32),
        old_per_token_logps if has_old else dummy, ref_per_token_logps if has_ref else dummy)
