"""CPU-side checks: the C-ABI library loads and exports what the header declares, the ctypes
structs match the C layout, and the host-side argument validation rejects bad inputs before
anything is launched (no compute calls here: there is no GPU)."""
import ctypes
import os
import re

import pytest
import torch

from ttt_tk_b200 import _lib, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_header_symbols():
    lib = _lib.lib()
    header = open(os.path.join(ROOT, "include", "ttt_mlp_b200.h")).read()
    declared = set(re.findall(r"\b(ttt_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert lib.ttt_b200_version() >= 1000
    assert lib.ttt_b200_last_error() is not None


def test_struct_layout_matches_header_field_order():
    header = open(os.path.join(ROOT, "include", "ttt_mlp_b200.h")).read()
    for struct, cls in (("ttt_b200_fwd_args", _lib.FwdArgs), ("ttt_b200_bwd_args", _lib.BwdArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                names.append(re.findall(r"([A-Za-z_0-9]+)\s*$", part.strip())[0])
        assert names == [f[0] for f in cls._fields_], struct
    assert ctypes.sizeof(_lib.FwdArgs) == 15 * 8 + 6 * 4 + 4 * 8
    assert ctypes.sizeof(_lib.BwdArgs) == 42 * 8 + 6 * 4


def test_null_args_rejected_without_launch():
    lib = _lib.lib()
    assert lib.ttt_b200_forward(None, None) == 1
    assert b"NULL" in lib.ttt_b200_last_error()
    a = _lib.FwdArgs()
    a.B, a.H, a.NC, a.checkpoint_group_size, a.num_checkpoints = 1, 1, 4, 3, 1   # needs 2 checkpoints
    assert lib.ttt_b200_forward(ctypes.byref(a), None) == 1
    assert b"ceil" in lib.ttt_b200_last_error()
    a.num_checkpoints = 2
    assert lib.ttt_b200_forward(ctypes.byref(a), None) == 1     # NULL tensors
    b = _lib.BwdArgs()
    b.B, b.H, b.NC, b.checkpoint_group_size, b.num_checkpoints = 1, 1, 0, 1, 0
    assert lib.ttt_b200_backward(ctypes.byref(b), None) == 1


def _fwd_args(B=1, H=2, NC=3, cgs=2, dev="cpu"):
    n = -(-NC // cgs)
    bf, f32 = torch.bfloat16, torch.float32
    z = lambda *s, dt=f32: torch.zeros(*s, dtype=dt, device=dev)
    return [z(B, H, NC, 64, 64, dt=bf), z(B, H, NC, 64, 64, dt=bf), z(B, H, NC, 64, 64, dt=bf),
            z(B, H, NC, 64, dt=bf), z(1, H, 1, 64), z(1, H, 1, 64),
            z(B, H, 64, 256), z(B, H, 1, 256), z(B, H, 256, 64), z(B, H, 1, 64),
            z(B, H, n, 64, 256), z(B, H, n, 1, 256), z(B, H, n, 256, 64), z(B, H, n, 1, 64),
            z(B, H, NC, 64, 64, dt=bf), cgs]


def test_forward_rejects_cpu_tensors_and_bad_shapes():
    args = _fwd_args()
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.ttt_forward(*args)
    bad = _fwd_args()
    bad[0] = torch.zeros(1, 2, 3, 64, 32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="head dimension"):
        ops.ttt_forward(*bad)
    bad = _fwd_args()
    bad[0] = torch.zeros(1, 2, 3, 32, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="mini-batch size"):
        ops.ttt_forward(*bad)
    bad = _fwd_args()
    bad[-1] = 0
    with pytest.raises(RuntimeError, match="checkpoint_group_size"):
        ops.ttt_forward(*bad)
    bad = _fwd_args()
    bad[-1] = 1          # would need 3 checkpoints, tensors hold 2
    with pytest.raises(RuntimeError, match="checkpoint tensors"):
        ops.ttt_forward(*bad)


def test_package_input_recipe_equals_the_oracles():
    from oracle import ttt_mlp as orc
    from ttt_tk_b200.synthetic import make_inputs
    a = orc.make_inputs(1, 2, 2, seed=3, eta_scale=0.5, backward=True)
    b = make_inputs(1, 2, 2, seed=3, eta_scale=0.5, backward=True)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k
