"""Seeded synthetic MoE workloads (inputs of the grouped-GEMM path), generated on the device.

They stand in for real activations / checkpoints: activations ~ N(0, 1) in bf16, weights
~ N(0, 0.02), both quantised to MXFP8 (E4M3 + one E8M0 scale per 32 K elements) with this
package's quantiser; routing is uniform or Zipf(s) over a seeded permutation of the experts,
top-k without replacement; gating probabilities are a softmax over each token's k logits.
Rows are grouped by expert with the routing kernels and every group is padded to ``m_aligned``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from . import moe, ops

# name -> (experts, K, N, tokens, top-k, routing)
CONFIGS: Dict[str, dict] = {
    # CPU-runnable reference case: E=4, hidden 256, fused gate|up N=1024, 512 tokens top-1
    "c1": dict(experts=4, k=256, n=1024, tokens=512, topk=1, routing="uniform"),
    # Mixtral-shape FC1
    "c2": dict(experts=8, k=4096, n=28672, tokens=16384, topk=2, routing="uniform"),
    # DeepSeek-V3-shape fine-grained FC1
    "c3": dict(experts=256, k=7168, n=4096, tokens=8192, topk=8, routing="zipf"),
    # DeepSeek-shape FC2 (input = FC1 output of c3)
    "c4": dict(experts=256, k=2048, n=7168, tokens=8192, topk=8, routing="zipf"),
}


@dataclass
class Routing:
    topk_ids: torch.Tensor  # [T, k] int32
    topk_prob: torch.Tensor  # [T, k] float32
    counts: torch.Tensor  # [E] int32
    padded_offsets: torch.Tensor  # [E] int32 END offsets
    dst_row: torch.Tensor  # [T * k] int32
    m_rows: int  # padded_offsets[-1]
    routed_rows: int  # T * k


def make_routing(tokens: int, experts: int, topk: int, routing: str, seed: int, device, m_aligned: int = 128, zipf_s: float = 1.2) -> Routing:
    g = torch.Generator(device=device).manual_seed(seed)
    if routing == "uniform":
        w = torch.ones(experts, device=device)
    elif routing == "zipf":
        rank = torch.arange(1, experts + 1, device=device, dtype=torch.float32)
        perm = torch.randperm(experts, generator=g, device=device)
        w = torch.empty(experts, device=device)
        w[perm] = rank.pow(-zipf_s)
    else:
        raise ValueError(f"unknown routing {routing!r}")
    ids = torch.multinomial(w.expand(tokens, experts), topk, replacement=False, generator=g).to(torch.int32)
    logits = torch.randn(tokens, topk, generator=g, device=device)
    prob = torch.softmax(logits, dim=-1)
    counts, offsets, dst = moe.route(ids, experts, m_aligned)
    m_rows = int(offsets[-1].item())
    return Routing(ids, prob, counts, offsets, dst, m_rows, tokens * topk)


def make_weights(experts: int, n: int, k: int, seed: int, device, std: float = 0.02, chunk: int = 8):
    """Random [E, n, k] weights ~ N(0, std), quantised to MXFP8.  Returns (b (n, k, E) view of
    float8_e4m3fn storage [E, n, k], sfb 6-D E8M0 tensor (32, 4, n/128, 4, rest_k, E))."""
    if n % 128 != 0:
        raise ValueError("n must be a multiple of 128 so that experts' scale blocks stack")
    g = torch.Generator(device=device).manual_seed(seed)
    b = torch.empty((experts, n, k), dtype=torch.float8_e4m3fn, device=device)
    sfb = ops.empty_sf(n, k, experts, device=device)
    sf_flat = torch.as_strided(sfb.view(torch.uint8), (sfb.numel(),), (1,))
    per_expert = sf_flat.numel() // experts
    for e0 in range(0, experts, chunk):
        e1 = min(e0 + chunk, experts)
        w = (torch.randn((e1 - e0) * n, k, generator=g, device=device) * std).to(torch.bfloat16)
        ops.quantize_mxfp8_out(w, b[e0:e1].view(-1, k), sf_flat[e0 * per_expert : e1 * per_expert])
        del w
    return b.permute(1, 2, 0), sfb


def make_activations(routing: Routing, k: int, seed: int, device):
    """Token activations ~ N(0,1) bf16 [T, k], scattered into the expert-grouped padded buffer
    (padding rows zero) and quantised.  Returns (x [T, k] bf16, a (M, k, 1) E4M3, sfa, prob (M,1,1))."""
    g = torch.Generator(device=device).manual_seed(seed)
    tokens, topk = routing.topk_ids.shape
    x = torch.randn(tokens, k, generator=g, device=device).to(torch.bfloat16)
    m = routing.m_rows
    xg = torch.empty((m, k), dtype=torch.bfloat16, device=device)
    prob = torch.empty((m,), dtype=torch.float32, device=device)
    moe.scatter_rows(x, routing.dst_row, xg, rows_per_src=topk, in_prob=routing.topk_prob.reshape(-1).contiguous(), out_prob=prob)
    moe.zero_pad_rows(xg, routing.counts, routing.padded_offsets, prob)
    a, sfa = ops.quantize_mxfp8(xg)
    del xg
    # the reference validates the stride of the unit dimension too: (K, 1, M*K)
    return x, torch.as_strided(a, (m, k, 1), (k, 1, m * k)), sfa, prob.view(m, 1, 1)


def make_problem(name_or_cfg, device="cuda", seed: int = 0, m_aligned: int = 128, with_weights: bool = True) -> dict:
    """All inputs of one grouped-GEMM call for a named configuration (or a dict with the same
    keys).  FLOPs are counted on true routed rows: ``2 * routed_rows * n * k``."""
    cfg = dict(CONFIGS[name_or_cfg]) if isinstance(name_or_cfg, str) else dict(name_or_cfg)
    e, k, n = cfg["experts"], cfg["k"], cfg["n"]
    routing = make_routing(cfg["tokens"], e, cfg["topk"], cfg["routing"], seed, device, m_aligned)
    x, a, sfa, prob = make_activations(routing, k, seed + 1, device)
    out = dict(cfg=cfg, routing=routing, x=x, a=a, sfa=sfa, prob=prob, padded_offsets=routing.padded_offsets,
               alpha=torch.ones(e, dtype=torch.float32, device=device), m_rows=routing.m_rows,
               flops=2.0 * routing.routed_rows * n * k)  # fmt: skip
    if with_weights:
        out["b"], out["sfb"] = make_weights(e, n, k, seed + 2, device)
    return out
