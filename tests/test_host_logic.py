"""CPU-only checks: the C-ABI library loads and exports every declared symbol, and the
operator classes validate their arguments with the reference's exception types."""

import ctypes
import logging
import os
import re

import pytest
import torch

import cudnn_frontend_b200 as cf
from cudnn_frontend_b200 import _build, _lib, api_base, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_loads_and_exports_every_declared_symbol():
    path = _build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/b200moe.h but not exported"
    assert set(declared) == set(_lib.EXPORTED_SYMBOLS)
    assert _lib.load().b200moe_abi_version() == _lib.ABI_VERSION == 7
    assert _lib.load().b200moe_workspace_bytes(256, _lib.WORKSPACE_DISCRETE) == 256 * 256
    assert _lib.load().b200moe_workspace_bytes(256, 0) == 0
    assert _lib.load().b200moe_workspace_bytes(256, _lib.WORKSPACE_DYNAMIC_SCHED) == 128
    assert ops.workspace_bytes(8, True, True) == 8 * 256 + 128


def test_c_abi_rejects_bad_arguments_without_touching_a_device():
    lib = _lib.load()
    args = _lib.GemmArgs()
    args.m_rows, args.n, args.k, args.num_experts = 128, 256, 128, 2
    assert lib.b200moe_fc1_swiglu(ctypes.byref(args), None) == _lib.E_NULL
    assert "required" in _lib.last_error()
    assert lib.b200moe_quantize_mxfp8(16, 4, 24, 24, 16, 16, None) == _lib.E_SHAPE  # cols % 16 != 0
    assert lib.b200moe_route(None, 0, 2000, 128, 16, 16, 16, 16, None) == _lib.E_SHAPE
    with pytest.raises(ValueError):
        _lib.check(_lib.E_SHAPE)
    with pytest.raises(NotImplementedError):
        _lib.check(_lib.E_UNSUPPORTED)
    with pytest.raises(RuntimeError):
        _lib.check(700)


def test_sf_shape_and_stride_follow_the_128x4_layout():
    shape, stride = ops.sf_shape_stride(300, 288, 2)
    assert shape == (32, 4, 3, 4, 3, 2)
    assert stride == (16, 4, 3 * 512, 1, 512, 3 * 3 * 512)


def test_tuple_dict_unpacks_and_indexes():
    t = api_base.TupleDict(a=1, b=None, c=3)
    x, y, z = t
    assert (x, y, z) == (1, None, 3)
    assert t[0] == 1 and t["c"] == 3 and t[2] == 3
    with pytest.raises(IndexError):
        t[3]


def _fc1_samples(m=256, n=256, k=128, e=2, d_dtype=torch.bfloat16):
    a = torch.empty((m, k, 1), dtype=torch.float8_e4m3fn)
    b = torch.empty((e, n, k), dtype=torch.float8_e4m3fn).permute(1, 2, 0)
    c = torch.empty((m, n, 1), dtype=torch.bfloat16)
    d = torch.empty((m, n // 2, 1), dtype=d_dtype)
    sfa = ops.empty_sf(m, k, 1, device="cpu")
    sfb = ops.empty_sf(n, k, e, device="cpu")
    offs = torch.zeros(e, dtype=torch.int32)
    alpha = torch.ones(e)
    return dict(sample_a=a, sample_b=b, sample_c=c, sample_d=d, sample_sfa=sfa, sample_sfb=sfb,
                sample_padded_offsets=offs, sample_alpha=alpha, sample_d_col=None)  # fmt: skip


def test_fc1_check_support_error_classes():
    ok = _fc1_samples()
    # sf_vec_size 16 with fp8 inputs is rejected like in the reference
    vec16 = dict(ok, sample_sfa=ops.empty_sf(256, 256, 1, device="cpu"), sample_sfb=ops.empty_sf(256, 256, 2, device="cpu"))
    with pytest.raises(ValueError, match="sf_vec_size"):
        cf.GroupedGemmSwigluSm100(**vec16, sf_vec_size=16).check_support()
    bad = dict(ok, sample_d=torch.empty((256, 100, 1), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="D must have shape"):
        cf.GroupedGemmSwigluSm100(**bad, sf_vec_size=32).check_support()
    bad = dict(ok, sample_sfd_row=ops.empty_sf(256, 128, 1, device="cpu"))
    with pytest.raises(ValueError, match="all None or all not None"):
        cf.GroupedGemmSwigluSm100(**bad, sf_vec_size=32).check_support()
    with pytest.raises(ValueError, match="m_aligned"):
        cf.GroupedGemmSwigluSm100(**ok, sf_vec_size=32, m_aligned=192).check_support()
    with pytest.raises(ValueError, match="cluster"):
        cf.GroupedGemmSwigluSm100(**ok, sf_vec_size=32, cluster_shape_mn=(3, 1)).check_support()
    # uint8 operands are raw packed FP4, as in the reference: the fp8 samples of this case then no longer fit (K
    # doubles and the scale tensors are too short)
    bad = dict(ok, sample_a=torch.empty((256, 128, 1), dtype=torch.uint8), sample_b=ok["sample_b"].view(torch.uint8))
    with pytest.raises(ValueError):
        cf.GroupedGemmSwigluSm100(**bad, sf_vec_size=32).check_support()
    bad = dict(ok, sample_a=torch.empty((256, 128, 1), dtype=torch.float8_e5m2))  # A and B must agree
    with pytest.raises(ValueError):
        cf.GroupedGemmSwigluSm100(**bad, sf_vec_size=32).check_support()
    bad = dict(ok, sample_a=torch.empty((128, 256, 1), dtype=torch.float8_e4m3fn).permute(1, 0, 2))
    with pytest.raises(ValueError, match="k-major"):
        cf.GroupedGemmSwigluSm100(**bad, sf_vec_size=32).check_support()
    # a valid configuration gets as far as the device check
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA"):
            cf.GroupedGemmSwigluSm100(**ok, sf_vec_size=32).check_support()
    op = cf.GroupedGemmSwigluSm100(**ok, sf_vec_size=32)
    with pytest.raises(RuntimeError, match="compile"):
        op.execute(None, None, None, None, None, None, None, None)


def test_fc2_requires_prob_and_one_weight_mode():
    m, n, k, e = 256, 256, 128, 2
    a = torch.empty((m, k, 1), dtype=torch.float8_e4m3fn)
    b = torch.empty((e, n, k), dtype=torch.float8_e4m3fn).permute(1, 2, 0)
    sfa, sfb = ops.empty_sf(m, k, 1, device="cpu"), ops.empty_sf(n, k, e, device="cpu")
    d = torch.empty((m, n, 1), dtype=torch.bfloat16)
    offs, alpha = torch.zeros(e, dtype=torch.int32), torch.ones(e)
    with pytest.raises(ValueError, match="prob_tensor is required"):
        cf.GroupedGemmQuantSm100(a, sfa, offs, alpha, d, sample_b=b, sample_sfb=sfb, sf_vec_size=32).check_support()
    with pytest.raises(ValueError, match="not both"):
        cf.grouped_gemm_quant_wrapper_sm100(a, sfa, offs, alpha, b_tensor=b, sfb_tensor=sfb, b_ptrs=torch.zeros(2, dtype=torch.int64))
    with pytest.raises(ValueError, match="Must provide"):
        cf.grouped_gemm_quant_wrapper_sm100(a, sfa, offs, alpha)
    prob = torch.ones((m, 1, 1))
    with pytest.raises(ValueError, match="stride"):  # the reference's layout is (n, l) with stride (1, n)
        cf.GroupedGemmQuantSm100(a, sfa, offs, alpha, d, sample_b=b, sample_sfb=sfb, sample_prob=prob, sf_vec_size=32,
                                 sample_bias=torch.empty((n, e), dtype=torch.bfloat16)).check_support()  # fmt: skip
    with pytest.raises(ValueError, match="bias"):
        cf.GroupedGemmQuantSm100(a, sfa, offs, alpha, d, sample_b=b, sample_sfb=sfb, sample_prob=prob, sf_vec_size=32,
                                 sample_bias=torch.empty((e, n), dtype=torch.int32).t()).check_support()  # fmt: skip
    with pytest.raises(ValueError, match="MMA tiler N"):
        cf.GroupedGemmQuantSm100(a, sfa, offs, alpha, d, sample_b=b, sample_sfb=sfb, sample_prob=prob, sf_vec_size=32,
                                 mma_tiler_mn=(256, 128)).check_support()  # fmt: skip


def test_pointer_tensors_are_validated():
    from cudnn_frontend_b200.grouped_gemm_quant import _require_pointer_tensor

    with pytest.raises(ValueError):
        _require_pointer_tensor(torch.zeros(4, dtype=torch.int32), "b_ptrs")
    with pytest.raises(ValueError):
        _require_pointer_tensor(torch.zeros(4, dtype=torch.int64), "b_ptrs")  # not on a CUDA device
    with pytest.raises(ValueError):
        _require_pointer_tensor([1, 2], "b_ptrs")


def test_experimental_warning_is_emitted_once_per_class(caplog):
    api_base._reset_experimental_api_warning_registry()
    ok = _fc1_samples()
    with caplog.at_level(logging.WARNING):
        cf.GroupedGemmSwigluSm100(**ok, sf_vec_size=32)
        cf.GroupedGemmSwigluSm100(**ok, sf_vec_size=32)
    msgs = [r for r in caplog.records if "experimental API" in r.getMessage()]
    assert len(msgs) == 1


def test_interleave_gate_up_matches_oracle():
    from oracle import mxfp8_oracle as orc

    g = torch.arange(3 * 64 * 4, dtype=torch.float32).reshape(3, 64, 4)
    u = -g
    w = cf.interleave_gate_up(g, u)
    assert torch.equal(w, torch.from_numpy(orc.interleave_gate_up(g.numpy(), u.numpy())))


def test_custom_ops_are_registered_with_mutation_schemas():
    from cudnn_frontend_b200 import ops  # noqa: F401  (registration happens at import)

    for name, mutated in (("fc1_swiglu", ("c", "d", "amax", "sfd_row")), ("fc2_quant", ("d", "amax", "sfd_row")), ("quantize_mxfp8", ("q", "sf"))):
        schema = getattr(torch.ops.b200moe, name).default._schema
        args = {a.name: a for a in schema.arguments}
        for m in mutated:
            assert args[m].alias_info is not None and args[m].alias_info.is_write, f"{name}.{m} must be declared mutable"
        assert not args["a" if name != "quantize_mxfp8" else "x"].alias_info


def test_fused_plan_places_every_routed_row_once_inside_its_expert_group():
    """plan_fused against a brute-force construction: on the owning rank, expert groups are padded to
    m_aligned, and inside a group the rows of source rank 0 come first, then rank 1, ..., each in the
    sender's own order."""
    import numpy as np
    import torch

    from cudnn_frontend_b200.ep_layer import plan_fused

    g, e, m_aligned = 4, 12, 8
    e_local = e // g
    rng = np.random.default_rng(5)
    ids = [rng.integers(0, e, size=rng.integers(20, 60)) for _ in range(g)]
    ids[2][:] = ids[2] % 5  # some experts get nothing from rank 2
    counts = np.stack([np.bincount(i, minlength=e) for i in ids])
    counts[:, 7] = 0  # an expert nobody routes to
    ids = [i[i != 7] for i in ids]
    plans = [plan_fused(torch.from_numpy(counts).to(torch.int32), r, m_aligned) for r in range(g)]

    total = counts.sum(0)
    padded = -(-total // m_aligned) * m_aligned
    seen = [dict() for _ in range(g)]
    for s in range(g):
        order = np.argsort(ids[s], kind="stable")  # compact local rows = stable grouping by expert
        local_row = np.empty_like(order)
        local_row[order] = np.arange(len(order))
        for slot, ex in enumerate(ids[s]):
            d = ex // e_local
            row = int(plans[s].delta[ex]) + int(local_row[slot])
            assert row not in seen[d]
            seen[d][row] = (s, slot, ex)
    for d in range(g):
        ends = np.cumsum(padded[d * e_local : (d + 1) * e_local])
        assert plans[d].padded_offsets.tolist() == ends.tolist()
        assert int(plans[0].m_rows_all[d]) == int(ends[-1])
        assert int(plans[0].rows_all[d]) == int(total[d * e_local : (d + 1) * e_local].sum()) == len(seen[d])
        start = 0
        for el in range(e_local):
            ex = d * e_local + el
            rows = sorted(r for r, v in seen[d].items() if v[2] == ex)
            assert rows == list(range(start, start + int(total[ex])))  # compact from the group start
            srcs = [seen[d][r][0] for r in rows]
            assert srcs == sorted(srcs)  # by source rank
            for s in range(g):  # and in the sender's order within a source
                slots = [seen[d][r][1] for r in rows if seen[d][r][0] == s]
                assert slots == sorted(slots)
            start = int(ends[el])


def test_unified_glu_api_argument_rules():
    """GroupedGemmGluSm100 / grouped_gemm_glu_wrapper_sm100: one of the two weight modes, known act_func."""
    m, n, k, e = 256, 256, 128, 2
    a = torch.empty((m, k, 1), dtype=torch.float8_e4m3fn)
    b = torch.empty((e, n, k), dtype=torch.float8_e4m3fn).permute(1, 2, 0)
    sfa, sfb = ops.empty_sf(m, k, 1, device="cpu"), ops.empty_sf(n, k, e, device="cpu")
    d = torch.empty((m, n // 2, 1), dtype=torch.bfloat16)
    offs, alpha = torch.zeros(e, dtype=torch.int32), torch.ones(e)
    with pytest.raises(ValueError, match="not both"):
        cf.GroupedGemmGluSm100(a, None, d, sfa, offs, alpha, None, sample_b=b, sample_sfb=sfb, num_experts=e, b_shape=(n, k),
                               b_dtype=torch.float8_e4m3fn)  # fmt: skip
    with pytest.raises(ValueError, match="Must provide"):
        cf.GroupedGemmGluSm100(a, None, d, sfa, offs, alpha, None)
    with pytest.raises(ValueError, match="act_func"):
        cf.GroupedGemmGluSm100(a, None, d, sfa, offs, alpha, None, sample_b=b, sample_sfb=sfb, sf_vec_size=32,
                               act_func="relu").check_support()  # fmt: skip
    with pytest.raises(ValueError, match="b_major"):
        cf.GroupedGemmGluSm100(a, None, d, sfa, offs, alpha, None, num_experts=e, b_shape=(n, k), b_dtype=torch.float8_e4m3fn,
                               sf_vec_size=32, b_major="x").check_support()  # fmt: skip
    with pytest.raises(ValueError, match="not both"):
        cf.grouped_gemm_glu_wrapper_sm100(a, sfa, offs, alpha, b_tensor=b, sfb_tensor=sfb, b_ptrs=torch.zeros(2, dtype=torch.int64))


def test_oracle_geglu_and_bias_follow_the_reference_formulas():
    import numpy as np

    from oracle import mxfp8_oracle as orc

    r = np.random.default_rng(3)
    c = (r.standard_normal((8, 128)) * 6).astype(np.float32)
    prob = r.random(8).astype(np.float32)
    d = orc.geglu_interleaved(c, prob)
    gate, up = c[:, :32], c[:, 32:64]
    g = np.minimum(gate, 7.0)
    u = np.clip(up, -7.0, 7.0)
    want = (u + 1.0) * g / (1.0 + np.exp(-1.702 * g.astype(np.float64))) * prob[:, None]
    np.testing.assert_allclose(d[:, :32], want, rtol=1e-6, atol=1e-6)
    offs = np.array([3, 8], dtype=np.int32)
    bias = r.standard_normal((128, 2)).astype(np.float32)
    cb = orc.add_bias(c, bias, offs)
    np.testing.assert_allclose(cb[:3], c[:3] + bias[:, 0], rtol=0, atol=0)
    np.testing.assert_allclose(cb[3:], c[3:] + bias[:, 1], rtol=0, atol=0)
    cb2 = orc.add_bias(c, bias, offs, row_scale=prob)
    np.testing.assert_allclose(cb2[3:], c[3:] + bias[:, 1][None, :] * prob[3:, None], rtol=1e-6)


def test_balanced_placement_fills_every_rank_and_evens_out_rows():
    import numpy as np

    from cudnn_frontend_b200.ep_layer import balanced_placement

    rng = np.random.default_rng(2)
    loads = (1000.0 / np.arange(1, 65) ** 1.2)[rng.permutation(64)]
    slot = balanced_placement(loads, 8)
    assert sorted(slot) == list(range(64))  # a permutation: 8 experts on each of the 8 ranks
    per_rank = np.zeros(8)
    for e, p in enumerate(slot):
        per_rank[p // 8] += loads[e]
    contiguous = loads.reshape(8, 8).sum(1)
    assert per_rank.max() / per_rank.mean() < contiguous.max() / contiguous.mean()
    # the heaviest expert alone is the floor of the busiest rank
    assert per_rank.max() <= max(loads.max(), per_rank.mean()) * 1.35
    assert balanced_placement(loads, 8) == slot  # deterministic
    with pytest.raises(ValueError):
        balanced_placement(loads[:63], 8)


def test_fp4_operands_are_validated_on_their_logical_shape():
    """float4_e2m1fn_x2 packs two elements per byte along K: the operator classes validate the element counts
    (python/cudnn/api_base.py:650-713), the scale-factor shapes follow sf_vec_size."""
    m, n, k, e = 256, 256, 256, 2
    a = torch.empty((m, k // 2, 1), dtype=torch.uint8).view(torch.float4_e2m1fn_x2)
    b = torch.empty((e, n, k // 2), dtype=torch.uint8).view(torch.float4_e2m1fn_x2).permute(1, 2, 0)
    assert api_base.TensorSpec.of(a, "a").logical().shape == (m, k, 1)
    assert api_base.TensorSpec.of(b, "b").logical().stride == (k, 1, n * k)
    sfa = ops.empty_sf(m, k, 1, device="cpu", dtype=torch.float8_e4m3fn, sf_vec=16)
    sfb = ops.empty_sf(n, k, e, device="cpu", dtype=torch.float8_e4m3fn, sf_vec=16)
    common = dict(sample_a=a, sample_b=b, sample_c=torch.empty((m, n, 1), dtype=torch.bfloat16), sample_sfa=sfa, sample_sfb=sfb,
                  sample_padded_offsets=torch.zeros(e, dtype=torch.int32), sample_alpha=torch.ones(e), sample_d_col=None)  # fmt: skip
    with pytest.raises(ValueError, match="fp16, bf16, or float32"):
        cf.GroupedGemmSwigluSm100(**common, sample_d=torch.empty((m, n // 2, 1), dtype=torch.float8_e4m3fn), sf_vec_size=16).check_support()
    with pytest.raises(NotImplementedError, match="float32"):  # the reference disables fp4 + sf_vec 16 + float32 D
        cf.GroupedGemmSwigluSm100(**common, sample_d=torch.empty((m, n // 2, 1), dtype=torch.float32), sf_vec_size=16).check_support()
    with pytest.raises(ValueError, match="SFA must have shape"):  # scale tensors made for 16 do not fit 32
        cf.GroupedGemmSwigluSm100(**common, sample_d=torch.empty((m, n // 2, 1), dtype=torch.bfloat16), sf_vec_size=32).check_support()
    if not torch.cuda.is_available():  # a valid NVFP4 configuration gets as far as the device check
        with pytest.raises(RuntimeError, match="CUDA"):
            cf.GroupedGemmSwigluSm100(**common, sample_d=torch.empty((m, n // 2, 1), dtype=torch.bfloat16), sf_vec_size=16).check_support()
    # the same operands as raw uint8 bytes (the reference's interpret_uint8_as_fp4x2) are the same configuration
    raw = dict(common, sample_a=a.view(torch.uint8), sample_b=b.view(torch.uint8))
    op = cf.GroupedGemmSwigluSm100(**raw, sample_d=torch.empty((m, n // 2, 1), dtype=torch.bfloat16), sf_vec_size=16)
    assert op.a.dtype == torch.float4_e2m1fn_x2 and op.b.dtype == torch.float4_e2m1fn_x2
    with pytest.raises(NotImplementedError, match="float32"):
        cf.GroupedGemmSwigluSm100(**raw, sample_d=torch.empty((m, n // 2, 1), dtype=torch.float32), sf_vec_size=16).check_support()
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA"):
            op.check_support()


def test_dswiglu_and_wgrad_check_support_error_classes():
    m, n, k, e = 256, 128, 128, 2
    a = torch.empty((m, k, 1), dtype=torch.float8_e4m3fn)
    b = torch.empty((e, n, k), dtype=torch.float8_e4m3fn).permute(1, 2, 0)
    c = torch.empty((m, 2 * n, 1), dtype=torch.bfloat16)
    d8 = torch.empty((m, 2 * n, 1), dtype=torch.float8_e4m3fn)
    sfa, sfb = ops.empty_sf(m, k, 1, device="cpu"), ops.empty_sf(n, k, e, device="cpu")
    offs, ones = torch.zeros(e, dtype=torch.int32), torch.ones(e)
    prob, dprob = torch.ones((m, 1, 1)), torch.zeros((m, 1, 1))
    sfd = dict(sample_sfd_row=ops.empty_sf(m, 2 * n, 1, device="cpu"), sample_sfd_col=ops.empty_sf(2 * n, m, 1, device="cpu"), sample_norm_const=torch.ones(1))
    args = (a, b, c, d8, d8, sfa, sfb, offs, ones, ones, prob, dprob)
    with pytest.raises(ValueError, match="epilogue operation"):
        cf.GroupedGemmDswigluSm100(*args, **sfd, sf_vec_size=32, epilogue_op="gelu")
    # accepted and without effect, as in the reference (its kernel never applies the lambda): every argument check
    # passes, and without a GPU the only complaint left is the missing device
    try:
        assert cf.GroupedGemmDswigluSm100(*args, **sfd, sf_vec_size=32, epilogue_op="relu").check_support()
    except RuntimeError as exc:
        assert "CUDA is not available" in str(exc)
    with pytest.raises(ValueError, match="D_row must be fp8"):  # fp8 operands take an fp8 D_row, as in the reference
        cf.GroupedGemmDswigluSm100(a, b, c, c, c, sfa, sfb, offs, ones, ones, prob, dprob, sf_vec_size=32).check_support()
    with pytest.raises(ValueError, match="C must have shape"):
        cf.GroupedGemmDswigluSm100(a, b, torch.empty((m, n, 1), dtype=torch.bfloat16), d8, d8, sfa, sfb, offs, ones, ones, prob, dprob, **sfd,
                                   sf_vec_size=32).check_support()  # fmt: skip
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA"):
            cf.GroupedGemmDswigluSm100(*args, **sfd, sf_vec_size=32).check_support()

    # weight gradient: A (m, T) and B (T, n) stored [n, T]; scale tensors (round_up(rows, 128), round_up(T / 32, 4))
    mw, nw, t = 384, 640, 640
    aw = torch.empty((mw, t), dtype=torch.float8_e4m3fn)
    bw = torch.empty((nw, t), dtype=torch.float8_e4m3fn).t()
    sa = torch.empty((384, 20), dtype=torch.uint8).view(torch.float8_e8m0fnu)
    sb = torch.empty((640, 20), dtype=torch.uint8).view(torch.float8_e8m0fnu)
    off = torch.tensor([256, 640], dtype=torch.int32)
    w = torch.empty((2, mw, nw), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="not both"):
        cf.GroupedGemmWgradSm100(aw, bw, sa, sb, off, sample_wgrad=w, num_experts=2)
    with pytest.raises(ValueError, match="contiguous along the tokens"):
        cf.GroupedGemmWgradSm100(aw, torch.empty((t, nw), dtype=torch.float8_e4m3fn), sa, sb, off, sample_wgrad=w, sf_vec_size=32).check_support()
    with pytest.raises(ValueError, match="sample_sfa must have shape"):
        cf.GroupedGemmWgradSm100(aw, bw, sb, sb, off, sample_wgrad=w, sf_vec_size=32).check_support()
    with pytest.raises(ValueError, match="wgrad_shape"):
        cf.GroupedGemmWgradSm100(aw, bw, sa, sb, off, num_experts=2, wgrad_shape=(mw, 2 * nw), wgrad_dtype=torch.bfloat16, sf_vec_size=32).check_support()
    with pytest.raises(ValueError, match="wgrad_ptrs is required"):
        cf.grouped_gemm_wgrad_wrapper_sm100(aw, bw, sa, sb, off, output_mode="discrete")
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA"):
            cf.GroupedGemmWgradSm100(aw, bw, sa, sb, off, sample_wgrad=w, sf_vec_size=32).check_support()
