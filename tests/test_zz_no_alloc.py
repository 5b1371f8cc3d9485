"""The workspace-free discrete-weight FC1 entry point against the regular one.

Some users of the library cannot allocate device memory when they call it (an inference server
that has already handed all free GPU memory to its own arena, a plugin that is given tensors but
no allocator, a loop that must never reach cudaMalloc).  ``b200moe_fc1_swiglu_discrete_noalloc``
serves them: it keeps the per-expert descriptor table in a fixed array inside the library instead
of in a caller workspace.  This test calls it through the C ABI several times in a row, with different
experts and weights each time (the array keeps the previous call's contents), and requires
bit-identical outputs to ``b200moe_fc1_swiglu`` given a caller workspace.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _problem(seed, groups, n, k):
    from cudnn_frontend_b200 import _lib, ops

    dev = "cuda"
    e = len(groups)
    valid, aligned, offs = orc.padded_end_offsets(groups, 128)
    a, b, sfa, sfb = H.gen_operands(seed, valid, n, k, e)
    H.zero_padding_rows(a, groups, aligned)
    keep = dict(
        a=H.dev_fp8(a),
        sfa=H.dev_sf(sfa, valid, k),
        b=[H.dev_fp8(b[i]) for i in range(e)],
        sfb=[H.dev_sf(sfb[i], n, k) for i in range(e)],
        offs=torch.from_numpy(offs).to(dev),
        alpha=torch.full((e,), 0.5, device=dev),
        prob=torch.rand(valid, device=dev) + 0.1,
    )
    keep["b_ptrs"] = torch.tensor([t.data_ptr() for t in keep["b"]], dtype=torch.int64, device=dev)
    keep["sfb_ptrs"] = torch.tensor([t.data_ptr() for t in keep["sfb"]], dtype=torch.int64, device=dev)

    def outputs():
        return dict(
            c=torch.zeros((valid, n), dtype=torch.bfloat16, device=dev),
            d=torch.zeros((valid, n // 2), dtype=torch.bfloat16, device=dev),
            amax=torch.full((e,), float("-inf"), device=dev),
        )

    def args(out, workspace, flags=0):
        g = _lib.GemmArgs()
        g.flags = flags
        g.a, g.sfa = keep["a"].data_ptr(), keep["sfa"].data_ptr()
        g.b_ptrs, g.sfb_ptrs = keep["b_ptrs"].data_ptr(), keep["sfb_ptrs"].data_ptr()
        g.padded_offsets, g.alpha, g.prob = keep["offs"].data_ptr(), keep["alpha"].data_ptr(), keep["prob"].data_ptr()
        g.c, g.d, g.amax = out["c"].data_ptr(), out["d"].data_ptr(), out["amax"].data_ptr()
        if workspace is not None:
            g.workspace, g.workspace_bytes = workspace.data_ptr(), workspace.numel()
        g.m_rows, g.n, g.k, g.num_experts = valid, n, k, e
        g.d_dtype = _lib.DTYPE_BF16
        return g

    ws = torch.zeros(ops.workspace_bytes(e, True), dtype=torch.uint8, device=dev)
    return keep, outputs, args, ws


def test_noalloc_entry_point_matches_workspace_entry_point_twice():
    from cudnn_frontend_b200 import _lib

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # the third call forces CTA-pair tiles: that mode also reads the scale-factor half of the descriptor table
    cases = ((71, [256, 0, 128], 512, 256, 0), (72, [128, 128, 384, 1, 200], 256, 384, 0), (74, [256, 0, 512], 512, 256, _lib.FLAG_TILE_PAIR))
    for seed, groups, n, k, flags in cases:
        keep, outputs, args, ws = _problem(seed, groups, n, k)
        ref, got = outputs(), outputs()
        rc = lib.b200moe_fc1_swiglu(ctypes.byref(args(ref, ws, flags)), stream)
        assert rc == 0, _lib.last_error()
        rc = lib.b200moe_fc1_swiglu_discrete_noalloc(ctypes.byref(args(got, None, flags)), stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert lib.b200moe_device_status(1) == 0
        assert torch.count_nonzero(ref["d"]) > 0
        for key in ("c", "d", "amax"):
            assert torch.equal(ref[key], got[key]), f"{key} differs (seed {seed})"
        del keep


def test_noalloc_entry_point_rejects_what_it_cannot_serve():
    from cudnn_frontend_b200 import _lib

    lib = _lib.load()
    keep, outputs, args, ws = _problem(73, [128], 256, 128)
    g = args(outputs(), None)
    g.num_experts = _lib.NOALLOC_MAX_EXPERTS + 1
    assert lib.b200moe_fc1_swiglu_discrete_noalloc(ctypes.byref(g), None) == _lib.E_SHAPE
    assert "at most" in _lib.last_error()
    g = args(outputs(), None)
    g.b, g.b_ptrs = keep["a"].data_ptr(), None  # dense weights are not what this entry point is for
    assert lib.b200moe_fc1_swiglu_discrete_noalloc(ctypes.byref(g), None) == _lib.E_NULL
