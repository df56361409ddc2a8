"""Times each kernel of a decode or prefill step alone, at a model's layer sizes.

    python -m edgelm_b200.kernel_bench --case decode  [--preset smollm2-135m] [--batch 8] [--ctx 1500]
    python -m edgelm_b200.kernel_bench --case prefill [--preset smollm2-135m] [--tokens 2048]
    ... [--only attn_prefill] [--layers 30] [--reps 5] [--plain]

Every kernel is launched once per layer on that layer's own weights and cache (so that weights
come from HBM as they do in a real step), the launches are captured in one CUDA graph, and the
graph is replayed `reps` times between two CUDA events: the figure is device time per launch
without host overhead.  `--plain` launches eagerly instead (one pass, no graph, no timing): the
form to run under a profiler, which sees one launch per layer.  Random weights; nothing here is
model code: it calls the same kernel wrappers the parts call.
"""
import argparse
import math
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", choices=["decode", "prefill"], required=True)
    ap.add_argument("--preset", default="smollm2-135m")
    ap.add_argument("--batch", type=int, default=8, help="decode: sequences")
    ap.add_argument("--ctx", type=int, default=1500, help="decode: cached tokens per sequence")
    ap.add_argument("--tokens", type=int, default=2048, help="prefill: new tokens of one sequence")
    ap.add_argument("--layers", type=int, default=None, help="layers' worth of distinct weights to cycle through")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--only", default=None, help="run only the kernels whose name contains this")
    ap.add_argument("--splits", type=int, default=0, help="decode: blocks per (sequence, kv head) of the attention")
    ap.add_argument("--no-fuse-norm", action="store_true", help="decode: the projections read a normalised input instead of computing the norm")
    ap.add_argument("--trace", action="store_true", help="prefill: clock stamps inside the tcgen05 attention kernel")
    ap.add_argument("--plain", action="store_true", help="eager launches, no graph and no timing (for profilers)")
    args = ap.parse_args(argv)

    from .csrc import ops as o
    from .presets import preset_config
    o.require_device()
    cfg = preset_config(args.preset)
    d = torch.device("cuda:0")
    D, nh, nkv, hd, I, V = (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                            cfg.intermediate_size, cfg.vocab_size)
    L = args.layers or cfg.num_hidden_layers
    QKV = (nh + 2 * nkv) * hd
    bf = torch.bfloat16
    decode = args.case == "decode"
    T = args.batch if decode else args.tokens
    B = args.batch if decode else 1
    ctx_len = args.ctx if decode else args.tokens

    def rn(*s, dt=bf):
        return (torch.randn(*s, device=d) * 0.05).to(dt)

    wq = [rn(QKV, D) for _ in range(L)]
    wo = [rn(D, nh * hd) for _ in range(L)]
    wg = [rn(I, D) for _ in range(L)]
    wu = [rn(I, D) for _ in range(L)]
    wd = [rn(D, I) for _ in range(L)]
    emb = rn(V, D)
    x = rn(T, D, dt=torch.float32)
    nw = torch.ones(D, device=d)
    h, qkv, att, mid = rn(T, D), rn(T, QKV), rn(T, nh * hd), rn(T, I)
    logits = torch.empty(B, V, device=d)
    pages_per = (ctx_len + 63) // 64 + 1
    n_pages = B * pages_per
    kc = [rn(n_pages, nkv, 64, hd) for _ in range(L)]
    vc = [rn(n_pages, nkv, 64, hd) for _ in range(L)]
    table = torch.arange(n_pages, dtype=torch.int32, device=d).view(B, pages_per).contiguous()
    seq = torch.arange(B, dtype=torch.int32, device=d)
    cos = torch.ones(cfg.max_position_embeddings, hd // 2, device=d)
    sin = torch.zeros(cfg.max_position_embeddings, hd // 2, device=d)
    err = torch.zeros(1, dtype=torch.int32, device=d)
    tok = torch.zeros(B, dtype=torch.int32, device=d)
    scale = 1.0 / math.sqrt(hd)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=d)
    flops = {}
    if decode:
        pos = torch.full((B,), ctx_len - 1, dtype=torch.int32, device=d)
        tokpos, tokseq = pos.clone(), seq.clone()
        splits = args.splits or min(16, max(1, (2 * 148 + B * nkv - 1) // (B * nkv)))
        po = torch.empty(B * nh * splits * hd, device=d)
        pm = torch.empty(B * nh * splits * 2, device=d)
        few = B <= 16
        cases = {
            "qkv_normed": lambda l: (o.gemv_mma(h, wq[l], qkv) if args.no_fuse_norm else o.gemv_mma(x, wq[l], qkv, norm_weight=nw, eps=1e-5)) if few else o.gemm_tc(h, wq[l], qkv, err),
            "rope_kv_append": lambda l: o.rope_kv_append(qkv, tokpos, tokseq, seq, table, cos, sin, kc[l], vc[l], nh, nkv, hd, err),
            "attn_decode": lambda l: o.attn_decode(qkv, att, kc[l], vc[l], table, seq, pos, B, nh, nkv, hd, scale, splits, po, pm),
            "o_proj_residual": lambda l: o.gemv_mma(att, wo[l], x, epilogue=o.EPI_RESIDUAL, residual=x) if few else o.gemm_tc(att, wo[l], x, err, epilogue=o.EPI_RESIDUAL, residual=x),
            "gate_up_swiglu_normed": lambda l: (o.gemv_mma(h, wg[l], mid, epilogue=o.EPI_SWIGLU, w2=wu[l]) if args.no_fuse_norm else o.gemv_mma(x, wg[l], mid, epilogue=o.EPI_SWIGLU, w2=wu[l], norm_weight=nw, eps=1e-5)) if few else o.gemm_tc(h, wg[l], mid, err, epilogue=o.EPI_SWIGLU, w2=wu[l]),
            "down_proj_residual": lambda l: o.gemv_mma(mid, wd[l], x, epilogue=o.EPI_RESIDUAL, residual=x) if few else o.gemm_tc(mid, wd[l], x, err, epilogue=o.EPI_RESIDUAL, residual=x),
            "rmsnorm": lambda l: o.rmsnorm(x, nw, 1e-5, h),
            "lm_head": lambda l: o.gemv_mma(h, emb, logits) if few else o.gemm_tc(h, emb, logits, err),
            "argmax": lambda l: o.argmax_rows(logits, tok),
        }
        print(f"decode: {args.preset}, batch {B}, context {ctx_len}, {splits} attention splits, {L} layers of weights")
    else:
        tokpos = torch.arange(T, dtype=torch.int32, device=d)
        tokseq = torch.zeros(T, dtype=torch.int32, device=d)
        nt = (T + 63) // 64
        t_seq, t_tok0 = mk([0] * nt), mk([i * 64 for i in range(nt)])
        t_ntok, t_pos0 = mk([min(64, T - i * 64) for i in range(nt)]), mk([i * 64 for i in range(nt)])
        nt2 = (T + 127) // 128
        u_seq, u_tok0 = mk([0] * nt2), mk([i * 128 for i in range(nt2)])
        u_ntok, u_pos0 = mk([min(128, T - i * 128) for i in range(nt2)]), mk([i * 128 for i in range(nt2)])
        flops = {"qkv_proj": 2 * T * QKV * D, "o_proj_residual": 2 * T * D * nh * hd, "gate_up_swiglu": 4 * T * I * D,
                 "down_proj_residual": 2 * T * D * I, "attn_prefill": 4 * nh * hd * T * (T + 1) / 2,
                 "attn_prefill_tc": 4 * nh * hd * T * (T + 1) / 2}
        cases = {
            "rmsnorm": lambda l: o.rmsnorm(x, nw, 1e-5, h),
            "qkv_proj": lambda l: o.gemm_tc(h, wq[l], qkv, err),
            "qkv_proj_rope_append": lambda l: o.gemm_tc_rope(h, wq[l], qkv, tokpos, tokseq, seq, table, cos, sin, kc[l], vc[l], nh, nkv, hd, err),
            "rope_kv_append": lambda l: o.rope_kv_append(qkv, tokpos, tokseq, seq, table, cos, sin, kc[l], vc[l], nh, nkv, hd, err),
            "attn_prefill": lambda l: o.attn_prefill_mma(qkv, att, kc[l], vc[l], table, seq, t_seq, t_tok0, t_ntok, t_pos0, nt, nh, nkv, hd, scale, max_keys=T),
            "attn_prefill_tc": lambda l: o.attn_prefill_tc(qkv, att, kc[l], vc[l], table, seq, u_seq, u_tok0, u_ntok, u_pos0, nt2, nh, nkv, hd, scale, err),
            "o_proj_residual": lambda l: o.gemm_tc(att, wo[l], x, err, epilogue=o.EPI_RESIDUAL, residual=x),
            "gate_up_swiglu": lambda l: o.gemm_tc(h, wg[l], mid, err, epilogue=o.EPI_SWIGLU, w2=wu[l]),
            "down_proj_residual": lambda l: o.gemm_tc(mid, wd[l], x, err, epilogue=o.EPI_RESIDUAL, residual=x),
        }
        flops["qkv_proj_rope_append"] = flops["qkv_proj"]
        if not o.gemm_tc_rope_takes(h, wq[0], qkv, kc[0], vc[0], cos, sin, hd):
            del cases["qkv_proj_rope_append"]
        if not o.attn_prefill_tc_takes(bf, hd):
            del cases["attn_prefill_tc"]
        elif args.trace:
            # one launch with clock stamps of a softmax warp per group, in the block with the most keys
            stamps = torch.zeros(o.ATTN_PREFILL_TC_TRACE_SHAPE, dtype=torch.int64, device=d)
            cases["attn_prefill_tc"](0)
            o.attn_prefill_tc_trace(stamps)
            cases["attn_prefill_tc"](0)
            o.attn_prefill_tc_trace(None)
            torch.cuda.synchronize()
            whole = stamps[-1].cpu()
            st = stamps[:-1].view(2, 64, 8).cpu()
            print("block: " + ", ".join(f"{nm} {(whole[i + 1] - whole[i]).item()}" for i, nm in enumerate(
                ["prologue", "wait for the kernel before", "key blocks", "last product and (m, l)", "merge and store", "last barrier"])))
            names = ["wait S", "scores to P", "wait P V", "(gap)", "rescale", "arrive"]
            for grp in range(2):
                n = int((st[grp, :, 0] > 0).sum())
                if n < 4:
                    continue
                body = st[grp, 2:n]   # steady state: without the first blocks
                per = (body[-1, 0] - body[0, 0]).item() / max(1, len(body) - 1)
                parts = [(body[:, i + 1] - body[:, i]).float().mean().item() for i in range(5)]
                print(f"group {grp}: {n} blocks, {per:.0f} clocks a block: " + ", ".join(f"{nm} {v:.0f}" for nm, v in zip(names, parts)))
                print(f"         issuer: P seen {(body[:, 6] - body[:, 5]).float().mean().item():.0f} clocks after the arrival, product issued {(body[:, 7] - body[:, 6]).float().mean().item():.0f} later;"
                      f" last block: arrival {(st[grp, n - 1, 5] - st[0, 0, 0]).item()}, seen {(st[grp, n - 1, 6] - st[0, 0, 0]).item()}, issued {(st[grp, n - 1, 7] - st[0, 0, 0]).item()}")
                print(f"         first stamp to last {(st[grp, n - 1, 5] - st[grp, 0, 0]).item()} clocks; starts of the blocks: "
                      + " ".join(str((st[grp, i, 0] - st[0, 0, 0]).item()) for i in range(min(n, 10))))
        print(f"prefill: {args.preset}, {T} tokens, {L} layers of weights")
    for name, fn in cases.items():
        if args.only and args.only not in name:
            continue
        for l in range(L):
            fn(l)
        torch.cuda.synchronize()
        if args.plain:
            print(f"{name:24s} launched {L} times")
            continue
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for l in range(L):
                fn(l)
        g.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.reps):
            g.replay()
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) * 1000 / (args.reps * L)
        extra = f"  {flops[name] / us / 1e6:8.1f} TFLOP/s" if name in flops else ""
        print(f"{name:24s} {us:8.2f} us{extra}")
    o.read_error_word(err)
    return 0


if __name__ == "__main__":
    sys.exit(main())
