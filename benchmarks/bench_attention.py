"""Device-timed flash-attention forward (tcgen05) vs torch SDPA on the same shapes.

    python benchmarks/bench_attention.py [--iters 20] [--only IDX] [--no-sdpa]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timeit(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", type=int, default=-1, help="index of the single shape to run (profiling captures)")
    ap.add_argument("--no-sdpa", action="store_true", help="skip the library comparison")
    ap.add_argument("--fwd-mode", type=int, default=0, help="0 = by size, 1 = one query tile per CTA, 2 = two tiles")
    ap.add_argument("--no-bwd", action="store_true", help="forward only")
    ap.add_argument("--bwd-mode", type=int, default=0, help="0 = second-generation backward kernels, 1 = first generation")
    args = ap.parse_args()
    from noeira_b200.ops import check_status
    from noeira_b200.ops.attention import flash_attention_backward, flash_attention_forward
    from noeira_b200.ops.attention import set_forward_mode
    set_forward_mode(args.fwd_mode)
    from noeira_b200.ops.attention import set_backward_mode
    set_backward_mode(args.bwd_mode)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    shapes = [  # B, S, Hq, Hkv, D, mask, frame
        (8, 1024, 12, 12, 64, None, 0),          # ViT tower
        (4, 4096, 16, 16, 128, "causal", 0),
        (1, 16384, 16, 4, 128, "block_causal", 256),  # world model, 64 frames x 256 tokens
        (8, 602, 8, 8, 64, None, 0),             # ACT encoder memory
        (4, 4096, 16, 16, 128, None, 0),
    ]
    if args.only >= 0:
        shapes = shapes[args.only: args.only + 1]
    for B, S, Hq, Hkv, D, mask, frame in shapes:
        q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
        k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        t = timeit(lambda: flash_attention_forward(q, k, v, mask=mask, frame=frame), args.iters, flush)
        check_status()
        frac = 1.0
        if mask == "causal":
            frac = 0.5
        elif mask == "block_causal":
            frac = 0.5 * (1 + frame / S)
        fl = 4.0 * B * Hq * S * S * D * frac
        row = {"shape": [B, S, Hq, Hkv, D], "mask": mask, "fwd_ms": round(t, 4), "fwd_tflops": round(fl / t / 1e9, 1)}
        try:
            if args.no_bwd:
                raise RuntimeError("skipped")
            o, lse = flash_attention_forward(q, k, v, mask=mask, frame=frame)
            do = torch.randn_like(o)
            tb = timeit(lambda: flash_attention_backward(q, k, v, o, lse, do, mask=mask, frame=frame), args.iters, flush)
            row.update(bwd_ms=round(tb, 4), bwd_tflops=round(2.5 * fl / tb / 1e9, 1))
        except Exception as e:  # noqa: BLE001
            row["bwd"] = str(e)[:60]
        if mask in (None, "causal") and not args.no_sdpa:
            qt, kt, vt = (x.permute(0, 2, 1, 3) for x in (q, k, v))
            if Hkv != Hq:
                kt, vt = kt.repeat_interleave(Hq // Hkv, 1), vt.repeat_interleave(Hq // Hkv, 1)
            tl = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=mask == "causal"),
                        args.iters, flush)
            row.update(sdpa_ms=round(tl, 4), sdpa_tflops=round(fl / tl / 1e9, 1))
        print(json.dumps(row))


if __name__ == "__main__":
    main()
