"""The C-ABI library: loads without a GPU, exports every symbol the header declares, the ctypes
mirror of the argument struct matches the C layout, and argument validation (which runs before
any CUDA call) returns the documented status codes.  No compute, no GPU."""
import ctypes as C
import os
import re
import subprocess

import pytest

from mllm_jax_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "mllm_grpo.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mllm_(?:grpo|ppo|lm_head)_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    lib = _lib.load()
    names = _declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mllm_grpo.h but not exported"
    assert set(_lib.EXPORTS) <= set(names)
    assert lib.mllm_grpo_abi_version() == 3


def test_ctypes_struct_matches_c_layout(tmp_path):
    """Compile a C program against the public header and compare sizeof/offsetof with the ctypes mirror."""
    fields = [f[0] for f in _lib.GrpoArgs._fields_]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "mllm_grpo.h"', "int main(void){",
             'printf("%zu\\n", sizeof(mllm_grpo_args));']
    lines += [f'printf("%zu\\n", offsetof(mllm_grpo_args, {f}));' for f in fields]
    lines += ["return 0;}"]
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{os.path.join(ROOT, 'include')}", str(src), "-o",
                    str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == C.sizeof(_lib.GrpoArgs)
    for f, off in zip(fields, out[1:]):
        assert getattr(_lib.GrpoArgs, f).offset == int(off), f


def test_value_struct_matches_c_layout(tmp_path):
    fields = [f[0] for f in _lib.PpoValueArgs._fields_]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "mllm_grpo.h"', "int main(void){",
             'printf("%zu\\n", sizeof(mllm_ppo_value_args));']
    lines += [f'printf("%zu\\n", offsetof(mllm_ppo_value_args, {f}));' for f in fields]
    lines += ["return 0;}"]
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{os.path.join(ROOT, 'include')}", str(src), "-o",
                    str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == C.sizeof(_lib.PpoValueArgs)
    for f, off in zip(fields, out[1:]):
        assert getattr(_lib.PpoValueArgs, f).offset == int(off), f


def test_lm_head_struct_matches_c_layout_and_validation(tmp_path, built_lib):
    fields = [f[0] for f in _lib.LmHeadArgs._fields_]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "mllm_grpo.h"', "int main(void){",
             'printf("%zu\\n", sizeof(mllm_lm_head_args));']
    lines += [f'printf("%zu\\n", offsetof(mllm_lm_head_args, {f}));' for f in fields]
    lines += ["return 0;}"]
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{os.path.join(ROOT, 'include')}", str(src), "-o",
                    str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == C.sizeof(_lib.LmHeadArgs)
    for f, off in zip(fields, out[1:]):
        assert getattr(_lib.LmHeadArgs, f).offset == int(off), f
    lib = _lib.load()
    a = _lib.LmHeadArgs()
    assert lib.mllm_lm_head_partials(C.byref(a), None) == 4  # struct size
    a.struct_size = C.sizeof(_lib.LmHeadArgs)
    assert lib.mllm_lm_head_partials(C.byref(a), None) == 2  # shape
    a.n_rows, a.vocab, a.hidden_dim, a.hidden_stride, a.weight_stride = 256, 1000, 128, 128, 128
    assert lib.mllm_lm_head_partials(C.byref(a), None) == 1  # null pointers
    a.hidden = a.weight = a.chosen_ids = a.partials = 0x1000
    a.hidden_dim = a.hidden_stride = a.weight_stride = 72
    assert lib.mllm_lm_head_partials(C.byref(a), None) == 7  # hidden size must be a multiple of 64
    assert lib.mllm_lm_head_splits(256, 151936) == 38 and lib.mllm_lm_head_splits(0, 5) == 0
    assert lib.mllm_lm_head_partials_bytes(256, 151936) == 38 * 256 * 16


def test_value_loss_validation(built_lib):
    a = _lib.PpoValueArgs()
    lib = _lib.load()
    assert lib.mllm_ppo_value_loss(C.byref(a), None) == 4  # struct size
    a.struct_size = C.sizeof(_lib.PpoValueArgs)
    assert lib.mllm_ppo_value_loss(C.byref(a), None) == 2  # shape
    a.n_seqs, a.seq_rows, a.scored_rows = 2, 4, 3
    assert lib.mllm_ppo_value_loss(C.byref(a), None) == 1  # null pointers
    assert lib.mllm_ppo_value_workspace_bytes(2, 4) == 24 and lib.mllm_ppo_value_workspace_bytes(0, 4) == 0


def _valid_args():
    a = _lib.GrpoArgs()
    a.struct_size = C.sizeof(_lib.GrpoArgs)
    a.n_seqs, a.seq_rows, a.scored_rows, a.vocab, a.row_stride = 2, 4, 3, 64, 64
    a.temperature, a.epsilon_low, a.epsilon_high = 1.0, 0.2, 0.3
    a.total_valid, a.grad_scale = 6.0, 1.0
    return a


def _status(name, a):
    return getattr(_lib.load(), name)(C.byref(a), None)


def test_validation_status_codes(built_lib):
    lib = _lib.load()
    assert lib.mllm_grpo_fwd(None, None) == 1  # NULL args
    a = _valid_args()
    a.struct_size = 8
    assert _status("mllm_grpo_fwd", a) == 4
    a = _valid_args()
    assert _status("mllm_grpo_fwd", a) == 1  # logits NULL
    for field, value in (("n_seqs", 0), ("vocab", -1), ("scored_rows", 5), ("row_stride", 63)):
        a = _valid_args()
        setattr(a, field, value)
        assert _status("mllm_grpo_fwd", a) == 2, field
    for field, value in (("temperature", 0.0), ("epsilon_low", -0.1), ("softcap", -1.0), ("temperature", float("nan"))):
        a = _valid_args()
        setattr(a, field, value)
        assert _status("mllm_grpo_bwd", a) == 3, field
    a = _valid_args()
    a.logits = 0x1001  # odd address: not even 2-byte aligned (validation never dereferences)
    a.chosen_ids = a.per_token_logps = 0x1000
    assert _status("mllm_grpo_logprobs", a) == 5
    a = _valid_args()
    a.n_seqs = 1 << 31
    assert _status("mllm_grpo_logprobs", a) == 8
    assert lib.mllm_grpo_status_string(2) == b"bad shape"
    assert lib.mllm_grpo_workspace_bytes(1000) == 4000
    assert lib.mllm_grpo_workspace_bytes(-5) == 0


def test_python_wrapper_raises_on_bad_status(built_lib):
    a = _valid_args()
    with pytest.raises(_lib.GrpoError) as e:
        _lib.call("mllm_grpo_fwd", a, 0)
    assert e.value.status == 1


def test_operators_refuse_cpu_tensors():
    import torch

    from mllm_jax_b200 import grpo_token_loss

    logits = torch.zeros(1, 3, 8, dtype=torch.bfloat16)
    ids = torch.zeros(1, 3, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA device only"):
        grpo_token_loss(logits, ids, ids, torch.zeros(1))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_gradient_buffer_layout_is_checked_on_the_host():
    """A gradient buffer whose strides differ from the logits' would be written out of bounds: refused."""
    import torch

    from mllm_jax_b200.ops import LossConfig, TokenLossProblem


    logits = torch.zeros(2, 3, 16, dtype=torch.bfloat16)
    prob = TokenLossProblem.__new__(TokenLossProblem)
    prob.logits = logits[:, :, :8]
    prob.dlogits = torch.zeros(2, 3, 8, dtype=torch.bfloat16)
    prob.B, prob.L, prob.T, prob.V, prob.row_stride = 2, 3, 3, 8, 16
    prob.vocab_start, prob.vocab_total, prob.cfg = 0, 8, LossConfig()
    prob.adv_per_token, prob.grad_scale, prob.total_valid = 0, 1.0, 1.0
    for name in ("chosen_ids", "mask", "advantages", "old_logps", "ref_logps", "total_valid_dev", "grad_scale_dev",
                 "per_token_logps", "token_entropy", "lse", "grad_coef", "loss", "loss_terms", "partials", "gathered",
                 "device_status", "peer_ptrs"):
        setattr(prob, name, None)
    prob.n_shards = prob.shard_rank = prob.exchange_epoch = 0
    with pytest.raises(ValueError, match="dlogits must match logits"):
        prob.args()
