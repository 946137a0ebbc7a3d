"""Runs the attention over a cache of latents (or, with --head-linear, the small products per head before and after it) of
given sizes three times, for ncu to capture one launch of a case that ends by itself:

    python -m research_2_b200.profiling.latent_case --heads 12 --rank 128 --rot 32 --entries 16 --rows 1024 &&
    ncu --set full --clock-control none -k regex:latent_attention -s 1 -c 1 -o latent \
        python -m research_2_b200.profiling.latent_case --heads 12 --rank 128 --rot 32 --entries 16 --rows 1024

With --time the case is timed inside a CUDA graph of 20 launches and microseconds per launch are printed.
"""
import argparse

import torch

from ..kernels import ops
from .kernel_cases import time_in_graph


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--rank", type=int, default=128, help="numbers of a latent (the value part of a cache row)")
    ap.add_argument("--rot", type=int, default=32, help="numbers of the rotated key part that all heads share")
    ap.add_argument("--dim", type=int, default=64, help="with --head-linear: a head's plain query part and its value size")
    ap.add_argument("--entries", type=int, default=16)
    ap.add_argument("--rows", type=int, default=1024, help="rows of every entry (1: a decode step)")
    ap.add_argument("--context", type=int, default=0, help="an entry's length after its rows (0: its rows)")
    ap.add_argument("--window", type=int, default=256)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--head-linear", action="store_true")
    ap.add_argument("--sinks", action="store_true", help="a learned term per head in the softmax's denominator")
    ap.add_argument("--time", action="store_true")
    args = ap.parse_args()
    dev, h, c, row, page = "cuda:0", args.heads, args.rank, args.rank + args.rot, args.page_size
    length = max(args.context, args.rows)
    t = args.entries * args.rows
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    queries = torch.randn(t, h * row, device=dev).bfloat16()
    mixed = torch.empty(t, h * c, device=dev, dtype=torch.bfloat16)
    if args.head_linear:
        proj = torch.randn(t, h * args.dim, device=dev).bfloat16()
        w_uk, w_uv = torch.randn(h * args.dim, c, device=dev).bfloat16(), torch.randn(h * args.dim, c, device=dev).bfloat16()
        out = torch.empty(t, h * args.dim, device=dev, dtype=torch.bfloat16)

        def fn():
            ops.head_linear(proj, args.dim, w_uk, False, queries, row, h, args.dim, c)
            ops.head_linear(mixed, c, w_uv, True, out, args.dim, h, c, args.dim)
    else:
        pages_each = -(-length // page)
        cache = torch.randn(args.entries * pages_each, page * row, device=dev).bfloat16().view(-1)
        tables = torch.arange(args.entries * pages_each, dtype=torch.int32, device=dev).view(args.entries, pages_each).contiguous()
        q_start = i32([i * args.rows for i in range(args.entries + 1)])
        row_entry = torch.arange(args.entries, dtype=torch.int32, device=dev).repeat_interleave(args.rows)
        positions = torch.arange(length - args.rows, length, dtype=torch.int32, device=dev).repeat(args.entries)
        seq_lens = i32([length] * args.entries)
        n_tiles = args.entries * -(-args.rows // 64)
        sinks = torch.randn(h, device=dev) if args.sinks else None

        def fn():
            ops.paged_attention(queries, cache, cache, page * row, page, args.entries * pages_each, tables, row_entry, positions, seq_lens,
                                h, 1, row, row ** -0.5, args.window, out=mixed, decode_only=args.rows == 1, max_context=length,
                                q_start=q_start, n_tiles=n_tiles, v_head_dim=c, values_in_keys=True, sinks=sinks)
    if args.time:
        print(f"{time_in_graph(fn):.1f} us a launch")
        return 0
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
