"""Single-kernel micro-benchmarks with roofline fractions.

    python -m chaoscontrol_b200.utils.kernel_bench --kernel gemm_resid --rows 262144 [--iters 20]

Times one kernel configuration with CUDA events (warm-up, L2 flushed between
iterations by writing a buffer larger than the 126 MB L2) and prints achieved
bytes/s and FLOP/s next to the measured peaks of ``MEASURED_PEAKS.json``
(fallback 6.65 TB/s / 1.59 PFLOP/s when the file is absent).  The same command
line is what the ncu captures under ``profiles/`` run.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..ops import _lib
from ..ops import gemm as G
from ..ops import lm_head as LH
from ..ops import scan as S

ROOT = Path(__file__).resolve().parents[2]


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "src": "fallback"}


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def build(kernel: str, R: int, D: int = 256, V: int = 16384, T: int = 512):
    """Returns (callable, algorithmic_bytes, flops)."""
    F = 2 * D
    x = _bf(R, D)
    ss = (x.float() ** 2).sum(-1)
    if kernel == "gemm_rowscale":           # packed projection
        w = _bf(4 * D, D, scale=0.06)
        out = torch.empty(R, 4 * D, dtype=torch.bfloat16, device="cuda")
        fn = lambda: G.gemm(x, w, epi=G.EPI_ROWSCALE, rowss=ss, inv_dim=1.0 / D, out=out)
        return fn, 2 * R * D + 2 * R * 4 * D, 2.0 * R * D * 4 * D
    if kernel == "gemm_resid":              # out_proj + residual + row ss
        w = _bf(D, D, scale=0.06)
        y = _bf(R, D)
        out = torch.empty_like(x)
        sso = torch.empty(R, dtype=torch.float32, device="cuda")
        fn = lambda: G.gemm(y, w, epi=G.EPI_RESID_SS, r1=x, ss_out=sso, out=out)
        return fn, 3 * 2 * R * D, 2.0 * R * D * D
    if kernel == "gemm_silu":
        w = _bf(F, D, scale=0.06)
        u = torch.empty(R, F, dtype=torch.bfloat16, device="cuda")
        f = torch.empty_like(u)
        fn = lambda: G.gemm(x, w, epi=G.EPI_ROWSCALE_SILU, rowss=ss, inv_dim=1.0 / D, out=u, c2=f)
        return fn, 2 * R * D + 2 * 2 * R * F, 2.0 * R * D * F
    if kernel == "gemm_dsilu":
        w = _bf(D, F, scale=0.06)
        u = _bf(R, F)
        out = torch.empty(R, F, dtype=torch.bfloat16, device="cuda")
        fn = lambda: G.gemm(x, w, b_mn=True, epi=G.EPI_DSILU, r1=u, rowss=ss, inv_dim=1.0 / D, out=out)
        return fn, 2 * R * D + 2 * 2 * R * F, 2.0 * R * D * F
    if kernel == "gemm_rmsbwd":
        w = _bf(F, D, scale=0.06)
        du = _bf(R, F)
        dres = _bf(R, D)
        out = torch.empty_like(x)
        fn = lambda: G.gemm(du, w, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss,
                            inv_dim=1.0 / D, out=out)
        return fn, 2 * R * F + 3 * 2 * R * D, 2.0 * R * D * F
    if kernel == "gemm_store":
        w = _bf(D, D, scale=0.06)
        out = torch.empty_like(x)
        fn = lambda: G.gemm(x, w, b_mn=True, out=out)
        return fn, 2 * 2 * R * D, 2.0 * R * D * D
    if kernel == "gemm_wgrad":
        dy = _bf(R, 4 * D)
        Ssp = G.pick_splits(4 * D, D, R)
        out = torch.empty(Ssp, 4 * D, D, dtype=torch.float32, device="cuda")
        fn = lambda: G.gemm(dy, x, a_mn=True, b_mn=True, splits=Ssp, out=out)
        return fn, 2 * R * 4 * D + 2 * R * D, 2.0 * R * D * 4 * D
    if kernel in ("scan_fwd", "scan_bwd"):
        B = R // T
        P = _bf(R, 4 * D)
        la = torch.zeros(D, device="cuda")
        if kernel == "scan_fwd":
            fn = lambda: S.scan_fused_fwd(P, la, None, B, T, D)
            return fn, 2 * R * 4 * D + 2 * 2 * R * D, 0.0
        y, h, _ = S.scan_fused_fwd(P, la, None, B, T, D)
        dy = _bf(R, D)
        dP = torch.empty_like(P)
        fn = lambda: S.scan_fused_bwd(P, la, None, h, dy, None, ss, 1.0 / D, 1e-6, B, T, D, dP=dP)
        return fn, 2 * R * 4 * D * 2 + 2 * 2 * R * D, 0.0
    if kernel in ("lmhead_lse", "lmhead_train"):
        W = _bf(V, D, scale=0.05)
        t = torch.randint(0, V, (R,), device="cuda")
        if kernel == "lmhead_lse":
            fn = lambda: LH.lm_head_lse(x, ss, W, t)
            return fn, 2 * R * D + 2 * V * D, 2.0 * R * D * V
        fn = lambda: LH.lm_head_train(x, ss, W, t, gscale=1.0 / R)
        # logits-sized GEMMs actually executed: one sweep = logits + dX, then logits + dW
        return fn, 2 * 2 * R * D + 2 * V * D, (4 if LH.ONE_SWEEP else 5) * 2.0 * R * D * V
    if kernel == "embed_bwd":
        from ..ops import trunk as T
        p = torch.arange(1, V + 1, dtype=torch.float64) ** -1.1
        tok = torch.multinomial(p / p.sum(), R, replacement=True).cuda()
        sc = torch.sort(tok, stable=True)
        dE = torch.empty(V, D, dtype=torch.float32, device="cuda")
        fn = lambda: T.embed_bwd(tok, x, V, sort_cache=sc, out=dE)
        return fn, 2 * R * D + 4 * V * D, 0.0
    raise SystemExit(f"unknown kernel {kernel}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--rows", type=int, default=262144)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--vocab", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--lmhead-parts", type=int, default=0, choices=[0, 2, 4],
                    help="epilogue width of the fused LM head: 2 = eight warps, 4 = sixteen (0: library default)")
    ap.add_argument("--gemm-cg", type=int, default=0, choices=[0, 1, 2],
                    help="1: one CTA per GEMM tile, 2: CTA pairs (cta_group::2); 0: library default")
    ap.add_argument("--gemm-debug", type=int, default=0,
                    help="stage-isolation bits of the GEMM kernel (1 no stores, 2 no epilogue math, 4 no TMEM "
                         "loads, 8 no MMAs): the output is wrong by design, only the time means something")
    ap.add_argument("--lmhead-debug", type=int, default=0,
                    help="stage-isolation bits of the fused LM head (1 no g-tile epilogue, 2 no second MMA, 4 no "
                         "logits MMA): wrong output by design, only the time means something")
    ap.add_argument("--lmhead-deep", type=int, default=-1, choices=[-1, 0, 1],
                    help="one-sweep LM-head training kernel: 1 = three W' stages with X in tensor memory, 0 = two "
                         "stages with X in shared memory (-1: library default)")
    ap.add_argument("--gemm-bres", type=int, default=-1, choices=[-1, 0, 1],
                    help="1: K <= 256 GEMMs keep their weight tile resident in shared memory (-1: library default)")
    ap.add_argument("--gemm-pres", type=int, default=-1, choices=[-1, 0, 1, 2, 3],
                    help="GEMM: CTA pairs with the weight tile resident (bit 1: K <= 256, bit 2: K <= 512)")
    ap.add_argument("--scan-poly", type=int, default=-1, choices=[-1, 0, 1, 2],
                    help="scan kernel arithmetic: 0 scalar, 1 scalar with FMA-pipe exponentials, 2 packed fp32x2")
    ap.add_argument("--gemm-l2pf", type=int, default=-2, choices=[-2, -1, 0, 1, 2, 3],
                    help="(-2: leave the library default) GEMM L2 prefetch bits: 1 = A tiles two tiles ahead, 2 = next tile's epilogue operands")
    a = ap.parse_args()
    if a.gemm_l2pf >= -1:
        _lib.lib().ccb_gemm_l2_prefetch(a.gemm_l2pf)
    if a.scan_poly >= 0:
        _lib.lib().ccb_scan_poly_exp(a.scan_poly)
    if a.gemm_pres >= 0:
        _lib.lib().ccb_gemm_pair_resident(a.gemm_pres)
    if a.gemm_bres >= 0:
        _lib.lib().ccb_gemm_resident_b(a.gemm_bres)
    if a.lmhead_deep >= 0:
        _lib.lib().ccb_lmhead_deep_ring(a.lmhead_deep)
    if a.lmhead_debug:
        _lib.lib().ccb_lmhead_debug(a.lmhead_debug)
    if a.gemm_debug:
        _lib.lib().ccb_gemm_debug(a.gemm_debug)
    if a.gemm_cg:
        _lib.lib().ccb_gemm_cta_group(a.gemm_cg)
    if a.lmhead_parts:
        _lib.lib().ccb_lmhead_epilogue_parts(a.lmhead_parts)
    torch.manual_seed(0)
    fn, nbytes, flops = build(a.kernel, a.rows, a.dim, a.vocab)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    _lib.assert_ok()
    times = []
    for _ in range(a.iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    ms = times[len(times) // 2]
    pk = peaks()
    out = {"kernel": a.kernel, "rows": a.rows, "lmhead_parts": a.lmhead_parts or None, "gemm_cg": a.gemm_cg or None, "gemm_debug": a.gemm_debug or None, "gemm_bres": a.gemm_bres if a.gemm_bres >= 0 else None, "gemm_l2pf": a.gemm_l2pf if a.gemm_l2pf >= -1 else None, "lmhead_debug": a.lmhead_debug or None, "lmhead_deep": a.lmhead_deep if a.lmhead_deep >= 0 else None, "scan_poly": a.scan_poly if a.scan_poly >= 0 else None, "gemm_pres": a.gemm_pres if a.gemm_pres >= 0 else None,
           "ms_median": ms, "ms_min": times[0],
           "GBps": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / pk["hbm_gbs"],
           "TFLOPs": flops / ms / 1e9, "frac_bf16_burst": flops / ms / 1e9 / pk["bf16_tflops"],
           "peaks": pk["src"]}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
