"""Throughput of the Kolorax design beside the closest existing model (Qwen3 dense) at equal size.

``python bench.py --design kolorax`` calls `main` here; the default workload of bench.py is untouched.
For each size, both models are built with seeded random weights at layer sizes that resemble a real
model's (same width, same number of layers, the dense feed-forward as wide as the experts a token
uses plus the shared one) and run through the engine's own loop (`Engine`: scheduler, captured decode
steps): a batch of prompts is prefilled, then decoded.  Times are wall clock around the engine loop with
a device synchronisation on both sides, after one untimed run of the same shape; prefill tokens per
second come from a run that generates one token, decode tokens per second from the extra time of a run
that generates N more.

The second part times the design's own kernels alone (CUDA events, inputs larger than L2 or an L2 flush
between iterations) against the bytes they must move or the operations they must do, next to the like
kernel of the dense model: the recurrence against the decode attention (both stream per-request state),
the grouped expert products against the dense feed-forward's product, layer norm against RMS norm.
"""
from __future__ import annotations

import json
import time
from types import SimpleNamespace

import torch

SIZES = {
    # width, layers, heads of the recurrent mixer (dim 64), attention heads, experts (top 4 of 16, 4 groups keep 2)
    "w1024": dict(width=1024, layers=8, ff=512, shared_ff=1024),
    "w2048": dict(width=2048, layers=8, ff=1024, shared_ff=2048),
}
VOCAB = 32768
TOP, EXPERTS, GROUPS, KEEP = 4, 16, 4, 2


def kolorax_config(width: int, layers: int, ff: int, shared_ff: int) -> dict:
    heads = width // 64
    mlp = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP, "groups": {"count": GROUPS, "keep": KEEP}},
           "expert": {"ff": ff, "limit": 7.0}, "shared": {"ff": shared_ff, "limit": 7.0}}
    wkv = {"type": "wkv", "mixer": {"heads": heads, "dim": 64, "decay_rank": 64}, "mlp": mlp}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 64, "kv_rank": 192, "scale": 128 ** -0.5,
                     "rot": {"base": 10000.0, "dims": 64}}}
    return {"architecture": "Kolorax", "vocab": VOCAB, "width": width, "residual_mult": 0.5, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": [lat if i % 4 == 3 else wkv for i in range(layers)], "loop": None}


def qwen3_config(width: int, layers: int, ff: int, shared_ff: int, max_len: int) -> dict:
    heads = width // 128
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=width, intermediate_size=TOP * ff + shared_ff,
                num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=max(1, heads // 4), head_dim=128,
                vocab_size=VOCAB, max_position_embeddings=max_len, rms_norm_eps=1e-6, rope_theta=1e4,
                tie_word_embeddings=False)


def run_engine(raw_cfg: dict, dtype: str, batch: int, prompt: int, new_tokens: int) -> dict:
    from .engine.engine import Engine, EngineOptions
    from .engine.loading import random_model
    from .engine.request import GenerationRequest
    from .models import config_from_dict
    from .ops import kernels as K
    from .sampling import SamplingParams
    cfg = config_from_dict(raw_cfg)
    model = random_model(cfg, 0, dtype=dtype)
    pages = batch * (-(-(prompt + new_tokens + 8) // 16) + 2)
    eng = Engine(model, options=EngineOptions(max_batch_size_limit=batch, kv_block_size=16, num_kv_blocks=pages,
                                              max_prefill_chunk_size=prompt, max_num_batched_tokens=max(8192, prompt),
                                              eos_token_ids=[]))
    g = torch.Generator().manual_seed(7)
    serial = [0]

    def once(n_new: int):
        reqs = []
        for _ in range(batch):
            toks = torch.randint(0, VOCAB, (prompt,), generator=g).tolist()
            serial[0] += 1
            reqs.append(GenerationRequest(f"b{serial[0]}", toks, SamplingParams(max_tokens=n_new, ignore_eos=True)))
        torch.cuda.synchronize()
        l0, t0 = K.LAUNCHES, time.perf_counter()
        for r in reqs:
            eng.add_request(r)
        while eng.has_unfinished_requests():
            eng.step()
        torch.cuda.synchronize()
        return time.perf_counter() - t0, K.LAUNCHES - l0
    once(new_tokens + 1)                      # kernels built, step shapes captured
    t_pre = min(once(1)[0] for _ in range(2))
    t_all, launches = min(once(new_tokens + 1) for _ in range(2))
    eng.runner.check_status()
    params = sum(t.numel() for t in model.weight_arena.tensors().values())
    del eng, model
    torch.cuda.empty_cache()
    return {"prefill_tok_s": round(batch * prompt / t_pre), "decode_tok_s": round(batch * new_tokens / max(t_all - t_pre, 1e-9)),
            "prefill_ms": round(t_pre * 1e3, 2), "decode_ms_per_step": round((t_all - t_pre) / new_tokens * 1e3, 3),
            "parameters_m": round(params / 1e6, 1), "launches": launches}


def _time(fn, iters: int = 10, flush=None) -> float:
    """Median microseconds of fn() by CUDA events; ``flush`` (a buffer larger than L2) is rewritten between runs."""
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def kernel_table(width: int, ff: int, batch: int, prompt: int, peaks: dict) -> list:
    """The design's kernels alone against their floors, and the dense model's like kernels at equal size."""
    from .ops import kernels as K
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, us, bytes_=0, flops=0, like=None):
        floor = max(bytes_ / hbm, flops / tflops) * 1e6
        rows.append({"kernel": name, "us": round(us, 1), "floor_us": round(floor, 2),
                     "of_floor": round(floor / us, 3) if us else None, "bound": "memory" if bytes_ / hbm >= flops / tflops else "tensor",
                     "like": like})
    heads, dim = width // 64, 64
    hd = heads * dim
    for label, n_seqs, q in (("prefill", batch, prompt), ("decode", batch * 8, 1)):
        T = n_seqs * q
        ctx = SimpleNamespace(cu_q=torch.arange(0, T + 1, q, dtype=torch.int32, device=dev), num_seqs=n_seqs,
                              state_slots=torch.arange(1, n_seqs + 1, dtype=torch.int32, device=dev),
                              seq_fresh=torch.zeros(n_seqs, dtype=torch.int32, device=dev))
        state = torch.zeros(n_seqs + 1, hd * dim + width, dtype=torch.float32, device=dev)
        rkvg = torch.randn(4, T, hd, device=dev).to(bf) * 0.1
        dlog = torch.randn(T, hd, device=dev)
        w0, u = torch.zeros(hd, device=dev), torch.randn(hd, device=dev)
        x, o = torch.randn(T, width, device=dev).to(bf), torch.empty(T, hd, device=dev)
        us = _time(lambda: K.wkv_scan(rkvg, dlog, w0, u, state, hd * dim, x, ctx, o, heads, dim), flush=flush)   # dim 64: its own size
        add(f"wkv_scan {label} ({n_seqs} x {q})", us, bytes_=3 * T * hd * 2 + 2 * T * hd * 4 + 2 * n_seqs * hd * dim * 4)
        # routed experts: gate|up with the activation, then down
        E, top = EXPERTS, TOP
        xa = torch.randn(T, width, device=dev).to(bf)
        z = torch.randn(T, E, device=dev)
        ids, wts = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, device=dev)
        K.moe_route(z, ids, wts, GROUPS, KEEP)
        n = T * top
        mt = K.moe_max_tiles(n, E, True)
        ints = [torch.empty(k, dtype=torch.int32, device=dev) for k in (E + 1, n, n, mt, mt, 1)]
        K.moe_plan(ids, E, *ints, True)
        plan = (ints[0], ints[3], ints[4], ints[5], mt)
        wg, wu = (torch.randn(E, ff, width, device=dev).to(bf) * 0.02 for _ in range(2))
        wd = torch.randn(E, width, ff, device=dev).to(bf) * 0.02
        act, outs = torch.empty(n, ff, dtype=bf, device=dev), torch.empty(n, width, device=dev)
        used = min(E, n)
        us = _time(lambda: K.moe_grouped(xa, ints[2], wg, wu, plan, act, 7.0, True), flush=flush)
        add(f"moe gate|up {label} ({n} rows)", us, bytes_=used * 2 * ff * width * 2 + n * (width + ff) * 2, flops=4 * n * ff * width)
        us = _time(lambda: K.moe_grouped(act, ints[2], wd, None, plan, outs, 0.0, True), flush=flush)
        add(f"moe down {label} ({n} rows)", us, bytes_=used * ff * width * 2 + n * (ff * 2 + width * 4), flops=2 * n * ff * width)
        # the dense model's like kernel: its gate|up product at the same number of operations
        inter = top * ff
        wdense = torch.randn(2 * inter, width, device=dev).to(bf) * 0.02
        yd = torch.empty(T, 2 * inter, dtype=bf, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        if T <= K.GEMM_TC_MAX_TOKENS:
            us = _time(lambda: K.gemm_tc(xa, wdense, yd, K.EPI_BF16, 4, st), flush=flush)
        else:
            us = _time(lambda: K.linear(xa, wdense, yd), flush=flush)
        add(f"dense gate|up {label} ({T} tokens)", us, bytes_=2 * inter * width * 2 + T * (width + 2 * inter) * 2,
            flops=4 * T * inter * width, like="moe gate|up")
        # norms
        res, dl = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev).to(bf)
        wn, bn, on = torch.ones(width, device=dev), torch.zeros(width, device=dev), torch.empty(T, width, dtype=bf, device=dev)
        if label == "prefill":
            us = _time(lambda: K.add_layer_norm(res, dl, wn, bn, 1e-6, on, None, 0.5), flush=flush)
            add(f"add_layer_norm ({T} rows)", us, bytes_=T * width * (4 + 4 + 2 + 2))
            us = _time(lambda: K.add_rms_norm(res, dl, wn, 1e-6, on), flush=flush)
            add(f"add_rms_norm ({T} rows)", us, bytes_=T * width * (4 + 4 + 2 + 2), like="add_layer_norm")
    return rows


def main(args, peaks: dict) -> int:
    out = {"design": "Kolorax", "beside": "Qwen3 dense at equal width, layers and feed-forward width per token",
           "dtype": args.dtype, "batch": args.batch, "prompt_len": args.prompt_len, "new_tokens": args.steps,
           "data": "synthetic token ids, seeded random weights", "peaks": peaks.get("source"), "sizes": {}}
    for name, size in SIZES.items():
        if args.design_sizes and name not in args.design_sizes.split(","):
            continue
        max_len = args.prompt_len + args.steps + 64
        ours = run_engine(kolorax_config(**size), args.dtype, args.batch, args.prompt_len, args.steps)
        dense = run_engine(qwen3_config(max_len=max_len, **size), args.dtype, args.batch, args.prompt_len, args.steps)
        out["sizes"][name] = {"shape": size, "kolorax": ours, "qwen3": dense,
                              "kernels": kernel_table(size["width"], size["ff"], args.batch, args.prompt_len, peaks)}
    print(json.dumps(out))
    return 0
