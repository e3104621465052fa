"""Kolorax on the device against the plain implementation in ``plain_kolorax.py``: every mechanism alone,
then whole models of several shapes through the replay session (whole prompts, decoding token by token,
portions down to two tokens, mixed batches with pages and state slots used again) and greedy generation
through the engine and its scheduler."""
import json
import os

import numpy as np
import pytest
import torch

import plain_kolorax as P
import replay_util as U

pytestmark = pytest.mark.gpu


def _wkv(heads, dim, rank=8):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def _lat(heads, dim, rot, vdim, rank, base=10000.0, scale=None, dims=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
                                                  "scale": scale or (dim + rot) ** -0.5,
                                                  "rot": {"base": base, "dims": rot if dims is None else dims}}}


def _moe(experts, top, count, keep, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}},
            "expert": {"ff": ff, "limit": limit}, "shared": shared}


def _cfg(layers, width=40, vocab=97, loop=None, mult=0.6, scale=1.5, eps=1e-5):
    return {"architecture": "Kolorax", "vocab": vocab, "width": width, "residual_mult": mult, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": layers, "loop": loop}


def _with(layer, mlp):
    return dict(layer, mlp=mlp)


CONFIGS = {
    # two kinds of mixer, a looped range run three times, experts in groups of two with one group left out
    "looped": _cfg([_with(_wkv(2, 24), _moe(6, 2, 3, 2, 24, 0.8, {"ff": 40, "limit": 1.7})),
                    _with(_lat(3, 16, 8, 24, 32), _moe(6, 2, 3, 2, 24, 0.8, {"ff": 40, "limit": 1.7})),
                    _with(_wkv(3, 16, 12), None)], loop={"start": 0, "stop": 2, "times": 3}),
    # attention first, no loop, one group (every expert may be chosen), one expert a token, no shared expert
    "plain_order": _cfg([_with(_lat(2, 24, 16, 16, 48, base=500.0, scale=0.3), _moe(4, 1, 1, 1, 32, 5.0)),
                         _with(_wkv(1, 48), _moe(8, 3, 8, 4, 16, 0.5, {"ff": 8, "limit": 0.9})),
                         _with(_lat(4, 8, 4, 8, 16), None)], width=48, vocab=131, mult=1.0, scale=1.0),
    # sizes that no fast path takes: a width that is no multiple of 8, a recurrent head of 20, five attention heads
    # over cache rows of 48, nine experts in three groups, part of the rotated vector left unturned
    "odd_sizes": _cfg([_with(_lat(5, 8, 16, 12, 32, base=77.0, dims=12), _moe(9, 4, 3, 3, 20, 1.2, {"ff": 12, "limit": 0.7})),
                       _with(_wkv(2, 20, 5), _moe(9, 4, 3, 3, 20, 1.2, {"ff": 12, "limit": 0.7}))],
                      width=36, vocab=50, loop={"start": 0, "stop": 2, "times": 2}, mult=0.8, scale=0.7),
    # recurrent layers only: no pages at all, only state slots
    "recurrent_only": _cfg([_with(_wkv(2, 32), _moe(4, 2, 2, 1, 16, 1.0, {"ff": 16, "limit": 1.0})),
                            _with(_wkv(5, 8), None)], loop={"start": 1, "stop": 2, "times": 2}),
}


def _model_dir(tmp_path, name, cfg, seed=1):
    w = P.random_weights(cfg, seed)
    raw = json.loads(json.dumps(cfg))
    for L in raw["layers"]:
        L["mixer"].pop("decay_rank", None)          # a folder need not say it: the tensor's shape does
    U.write_model_dir(str(tmp_path / name), raw, {k: v.float() for k, v in w.items()}, torch.bfloat16)
    return str(tmp_path / name), w


def _session(model_dir, dtype, max_tokens, block=16, max_requests=4):
    from firefly_b200.replay import ReplaySession
    return ReplaySession(model_dir, dtype=dtype, max_tokens=max_tokens, block_size=block, max_requests=max_requests)


def _compare_most(got, plain, tol, what, frac=0.97):
    """Every row within 8 tol, and ``frac`` of the rows within tol (a router's close call may move a row in bfloat16)."""
    errs = sorted(U.rel_err(row, plain[rid.split("#")[0]][pos]) for (rid, pos), row in got.rows.items())
    assert errs, what
    assert errs[-1] <= 8 * tol and errs[int(frac * (len(errs) - 1))] <= tol, \
        f"{what}: worst {errs[-1]:.3e}, {frac:.0%} quantile {errs[int(frac * (len(errs) - 1))]:.3e}, tol {tol:g}"


def _check(got, plain, dtype, what):
    if dtype == "float32":
        U.compare(got, plain, U.TOL[dtype], what)
    else:
        _compare_most(got, plain, U.TOL[dtype], what)


# ------------------------------------------------------------------ whole models, every cutting --
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_replay_in_every_cutting_matches_the_plain_model(tmp_path, name, dtype):
    cfg = CONFIGS[name]
    model_dir, w = _model_dir(tmp_path, name, cfg)
    reqs = U.make_requests(cfg["vocab"], [70, 3, 45, 1, 33, 58], 5)
    plain = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    twice = dict(reqs, **{"r0#2": reqs["r0"], "r4#2": reqs["r4"]})       # a request once more, on pages used before
    for label, steps in (("whole", U.trace_whole(reqs)), ("decode", U.trace_tail_decode(reqs, tail=40)),
                         ("portions", U.trace_portions(reqs, sizes=(17, 5, 2, 9, 2, 31, 3, 2))),
                         ("mixed", U.trace_mixed(twice, seed=3, max_live=4, sizes=(13, 2, 7, 21, 3, 2, 16)))):
        sess = _session(model_dir, dtype, U.peak_tokens(steps), block=16 if label != "portions" else 8)
        got = U.run_trace(sess, steps)
        _check(got, plain, dtype, f"{name}/{dtype}/{label}")
        sess.cache.check()
        assert not sess.cache.live


def test_the_layers_stream_matches_after_every_run(tmp_path):
    cfg = CONFIGS["looped"]
    model_dir, w = _model_dir(tmp_path, "stream", cfg)
    toks = U.make_requests(cfg["vocab"], [21], 8)["r0"]
    _, want = P.forward(cfg, w, toks, return_layers=True)
    sess = _session(model_dir, "float32", 64)
    got = []
    sess.model.after_run = lambda i, res, pending: got.append(res.detach().cpu().double().clone())
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": ["a"]})
    assert len(got) == len(P.layer_runs(cfg)) == 7
    for i, g in enumerate(got):
        assert float((g - want[i]).abs().max()) < 2e-5 * float(want[i].abs().max()), f"after run {i}"


# ------------------------------------------------------------------ mechanisms alone --
def _one_layer(tmp_path, layer, width=40, dtype="float32", seed=2, max_tokens=1024, block=16):
    cfg = _cfg([layer], width=width)
    model_dir, w = _model_dir(tmp_path, "one", cfg, seed)
    sess = _session(model_dir, dtype, max_tokens, block=block)
    return cfg, w, sess


def _step_context(sess, seqs):
    """A StepContext for sequences given as (request id, new tokens): admits, grows, builds."""
    from firefly_b200.engine.runner import StepEntry
    entries = []
    for rid, n in seqs:
        rc = sess.live.get(rid) or sess.cache.admit(rid)
        sess.live[rid] = rc
        assert sess.cache.grow(rc, rc.num_tokens + n)
        entries.append(StepEntry(rc, [0] * n, []))
    return sess.runner.build_context(entries), entries


def _advance(sess, entries):
    for e in entries:
        sess.cache.advance(e.cache, len(e.tokens))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wkv_mixer_alone_whole_then_in_portions_and_token_by_token(tmp_path, dtype):
    layer = _with(_wkv(3, 24, 12), None)
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(0)
    x = torch.randn(57, 40, generator=g).to(tdt)
    want, _ = P.wkv_mixer(x.double(), w, "l0.mix", 3, 24, cfg["norm"]["eps"])
    mixer = sess.model.blocks[0].mixer
    tol = 2e-5 if dtype == "float32" else 3e-2
    for cuts in ([57], [20, 2, 1, 1, 30, 3], [1] * 57):
        rid = f"r{len(cuts)}"
        rows, p = [], 0
        for n in cuts:
            ctx, entries = _step_context(sess, [(rid, n)])
            rows.append(mixer.forward(x[p:p + n].cuda().contiguous(), ctx, 0, True).float().cpu())
            _advance(sess, entries)
            p += n
        got = torch.cat(rows).double()
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts
        sess.cache.free(sess.live.pop(rid))        # the slot goes to the next cutting, which must start from zero


def test_wkv_state_of_a_freed_slot_does_not_leak_and_batches_equal_requests_alone(tmp_path):
    layer = _with(_wkv(2, 32), None)
    cfg, w, sess = _one_layer(tmp_path, layer)
    g = torch.Generator().manual_seed(1)
    xs = {rid: torch.randn(n, 40, generator=g) * 2 for rid, n in (("a", 9), ("b", 1), ("c", 30), ("d", 2))}
    want = {rid: P.wkv_mixer(x.double(), w, "l0.mix", 2, 32, cfg["norm"]["eps"])[0] for rid, x in xs.items()}
    mixer = sess.model.blocks[0].mixer
    for rounds in range(2):                       # the second round runs on slots the first one used
        ctx, entries = _step_context(sess, [(rid, x.shape[0]) for rid, x in xs.items()])
        order = [e.cache.request_id for e in sorted(entries, key=lambda e: 0 if len(e.tokens) == 1 else 1)]
        got = mixer.forward(torch.cat([xs[r] for r in order]).cuda(), ctx, 0, True).cpu().double()
        p = 0
        for r in order:
            n = xs[r].shape[0]
            assert float((got[p:p + n] - want[r]).abs().max()) < 2e-5 * float(want[r].abs().max()), (rounds, r)
            p += n
        for rid in xs:
            sess.cache.free(sess.live.pop(rid))


def _standout_inputs(w, p, T, width, far, query, heads, dim, rot, rank, scale, eps, seed):
    """Random inputs, except that the row `query` is solved for so that the plain part of its first two
    heads' queries points along the key of row `far`, with a score about 30 above the others: an attention
    that loses that one key among hundreds gives another result."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, width, generator=g) * 0.5
    dkv = w[f"{p}.dkv"] @ x[far].double()
    c = P.rms_unit(dkv[:rank], eps) * w[f"{p}.dkv.norm"]
    k = (w[f"{p}.uk"] @ c).view(heads, dim)[:2]
    beta = 30.0 / (scale * (k * k).sum(-1, keepdim=True))
    rows = w[f"{p}.q"].view(heads, dim + rot, width)[:2, :dim].reshape(-1, width)
    x[query] = (torch.linalg.pinv(rows) @ (beta * k).reshape(-1)).float()
    return x


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 255, 256])
def test_latent_attention_alone_sees_a_far_key_in_prompts_and_in_decoding(tmp_path, dtype, far):
    layer = _with(_lat(3, 16, 8, 24, 32, base=100.0, scale=0.9), None)
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype)
    mx = layer["mixer"]
    kw = dict(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=32, scale=mx["scale"], base=100.0, eps=cfg["norm"]["eps"])
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    T = 420
    x = _standout_inputs(w, "l0.mix", T, 40, far, T - 1, 3, 16, 8, 32, mx["scale"], cfg["norm"]["eps"], far).to(tdt)
    want, _ = P.latent_attention_mixer(x.double(), w, "l0.mix", torch.arange(T), **kw)
    lost, _ = P.latent_attention_mixer(torch.cat([x[:far], x[far + 1:]]).double(), w, "l0.mix",
                                       torch.cat([torch.arange(far), torch.arange(far + 1, T)]), **kw)
    assert float((lost[-1] - want[-1]).abs().max()) > 0.1 * float(want[-1].abs().max())      # the test can see the key
    mixer = sess.model.blocks[0].mixer
    tol = 2e-5 if dtype == "float32" else 4e-2
    for cuts in ([T], [T - 1, 1], [far + 1, T - far - 3, 2], [300, 100, 17, 1, 1, 1]):
        rid, rows, p = f"r{len(cuts)}", [], 0
        for n in cuts:
            ctx, entries = _step_context(sess, [(rid, n)])
            rows.append(mixer.forward(x[p:p + n].cuda().contiguous(), ctx, 0, True).float().cpu())
            _advance(sess, entries)
            p += n
        got = torch.cat(rows).double()
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts
        assert float((got[-1] - want[-1]).abs().max()) <= tol * float(want[-1].abs().max()), cuts
        sess.cache.free(sess.live.pop(rid))


def test_latent_attention_in_a_batch_of_unequal_requests_on_reused_pages(tmp_path):
    layer = _with(_lat(2, 24, 16, 16, 48, base=50.0, scale=0.4), None)
    cfg, w, sess = _one_layer(tmp_path, layer, max_tokens=512, block=8)
    kw = dict(heads=2, dim=24, rot_dim=16, vdim=16, kv_rank=48, scale=0.4, base=50.0, eps=cfg["norm"]["eps"])
    g = torch.Generator().manual_seed(4)
    for rounds in range(3):
        xs = {rid: torch.randn(n, 40, generator=g) for rid, n in (("a", 70), ("b", 1), ("c", 129), ("d", 2))}
        want = {rid: P.latent_attention_mixer(x.double(), w, "l0.mix", torch.arange(x.shape[0]), **kw)[0] for rid, x in xs.items()}
        mixer = sess.model.blocks[0].mixer
        # first portions together, then the rest beside each other's single tokens
        done = {rid: 0 for rid in xs}
        for take in ({"a": 33, "b": 1, "c": 64, "d": 1}, {"a": 36, "c": 1, "d": 1}, {"a": 1, "c": 64}):
            seqs = [(rid, n) for rid, n in take.items()]
            ctx, entries = _step_context(sess, seqs)
            order = [e.cache.request_id for e in sorted(entries, key=lambda e: 0 if len(e.tokens) == 1 else 1)]
            xin = torch.cat([xs[r][done[r]:done[r] + take[r]] for r in order])
            got = mixer.forward(xin.cuda(), ctx, 0, True).cpu().double()
            p = 0
            for r in order:
                ref = want[r][done[r]:done[r] + take[r]]
                assert float((got[p:p + take[r]] - ref).abs().max()) < 3e-5 * float(want[r].abs().max()), (rounds, r)
                p += take[r]
                done[r] += take[r]
            _advance(sess, entries)
        for rid in xs:
            sess.cache.free(sess.live.pop(rid))
        sess.cache.check()


@pytest.mark.parametrize("shape", [(6, 2, 3, 2), (8, 3, 8, 4), (4, 1, 1, 1), (12, 4, 2, 1), (5, 5, 1, 1)])
def test_router_choice_and_weights(shape):
    from firefly_b200.ops import kernels as K
    E, top, count, keep = shape
    g = torch.Generator().manual_seed(E * 7 + top)
    z = (torch.randn(64, E, generator=g) * 2).float()
    ids = torch.empty(64, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(64, top, dtype=torch.float32, device="cuda")
    K.moe_route(z.cuda(), ids, wts, count, keep)
    for t in range(64):
        chosen, w = P.route(z[t].double(), top, count, keep)
        assert ids[t].tolist() == chosen, t
        assert torch.allclose(wts[t].cpu().double(), w, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens", [1, 5, 150])
def test_experts_alone(tmp_path, dtype, tokens):
    mlp = _moe(6, 2, 3, 2, 24, 0.8, {"ff": 40, "limit": 1.7})
    cfg, w, sess = _one_layer(tmp_path, _with(_wkv(1, 8), mlp), dtype=dtype)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(tokens)
    x = (torch.randn(tokens, 40, generator=g) * 1.5).to(tdt)      # large enough for the clamps to act
    want = P.moe(x.double(), w, "l0.mlp", mlp)
    ctx, _ = _step_context(sess, [("a", tokens)])
    ff = sess.model.blocks[0].feed_forward
    got = ff.forward(x.cuda(), ctx).cpu().double()
    err = (got - want).abs().max(dim=1).values / want.abs().max()
    if dtype == "float32":
        assert float(err.max()) < 2e-5
    else:
        assert float(err.sort().values[int(0.95 * (tokens - 1))]) < 3e-2
    if dtype == "bfloat16":
        # the tensor-core grouped product against the plain one: the same sums in another order
        from firefly_b200.ops import kernels as K
        K.MOE_FORCE_PLAIN = True
        try:
            plain = ff.forward(x.cuda(), ctx).cpu().double()
        finally:
            K.MOE_FORCE_PLAIN = False
        assert float((got - plain).abs().max()) < 1e-2 * float(want.abs().max())
    # added into the stream times a multiplier
    res = torch.randn(tokens, 40, generator=g).cuda()
    before = res.clone()
    assert ff.forward(x.cuda(), ctx, accumulate_into=res, residual_scale=0.25) is None
    assert torch.allclose(res.cpu().double(), before.cpu().double() + 0.25 * got, rtol=1e-4, atol=1e-5)


def test_layer_norm_and_loop_input_alone(tmp_path):
    cfg = CONFIGS["looped"]
    model_dir, w = _model_dir(tmp_path, "ln", cfg)
    sess = _session(model_dir, "float32", 64)
    ctx, _ = _step_context(sess, [("a", 11)])
    g = torch.Generator().manual_seed(3)
    res, delta = torch.randn(11, 40, generator=g) * 3 + 1, torch.randn(11, 40, generator=g)
    r = res.cuda()
    norm = sess.model.blocks[0].norms[1]
    got = norm.forward(r, delta.cuda(), ctx, delta_scale=0.6)
    summed = res.double() + 0.6 * delta.double()
    assert torch.allclose(r.cpu().double(), summed, atol=1e-6)
    want = P.layer_norm(summed, w["l0.norm2"], w["l0.norm2.b"], cfg["norm"]["eps"])
    assert float((got.cpu().double() - want).abs().max()) < 1e-5
    rows = torch.tensor([7, 2], dtype=torch.int32, device="cuda")
    got = sess.model.final_norm.forward(r, None, ctx, tag="t", row_idx=rows)
    want = P.layer_norm(summed[[7, 2]], w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"])
    assert float((got.cpu().double() - want).abs().max()) < 1e-5
    x0 = torch.randn(11, 40, generator=g)
    out, pending = sess.model.junctions[0].forward(r, None, ctx, x0.cuda(), 2)
    want = torch.cat([summed, x0.double()], dim=-1) @ w["loop.in"].T + w["loop.step"][2]
    assert pending is None and float((out.cpu().double() - want).abs().max()) < 1e-4


# ------------------------------------------------------------------ long decoding, generation --
def test_long_decoding_keeps_state_and_cache(tmp_path):
    cfg = CONFIGS["plain_order"]
    model_dir, w = _model_dir(tmp_path, "long", cfg, seed=4)
    toks = U.make_requests(cfg["vocab"], [200], 2)["r0"]
    plain = {"r0": P.forward(cfg, w, toks).numpy()}
    steps = U.trace_tail_decode({"r0": toks}, tail=190)
    sess = _session(model_dir, "float32", U.peak_tokens(steps), block=8)
    U.compare(U.run_trace(sess, steps), plain, U.TOL["float32"], "long decoding")


@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_through_the_engine(tmp_path, graphs):
    from firefly_b200 import LLM
    cfg = CONFIGS["looped"]
    model_dir, w = _model_dir(tmp_path, "gen", cfg, seed=6)
    prompts = [v for v in U.make_requests(cfg["vocab"], [19, 3, 41, 8, 27], 11).values()]
    llm = LLM(model_dir, dtype="float32", max_batch_size_limit=3, kv_block_size=8, num_kv_blocks=40,
              max_prefill_chunk_size=16, eos_token_ids=[], use_cuda_graphs=graphs)
    outs = llm.generate(prompts, max_tokens=10, ignore_eos=True)
    llm.engine.cache.check()
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        rows = P.forward(cfg, w, list(p) + o[:-1])
        for i, tok in enumerate(o):
            row = rows[len(p) - 1 + i]
            top2 = torch.topk(row, 2).values
            assert tok == int(row.argmax()) or float(top2[0] - top2[1]) < 1e-4 * float(row.abs().max()), (i, tok)


def test_the_command_line_generates_from_a_folder_and_from_a_configuration(tmp_path):
    import subprocess
    import sys
    cfg = CONFIGS["recurrent_only"]
    model_dir, _ = _model_dir(tmp_path, "cli", cfg)
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "bin", "firefly")
    out = subprocess.run([sys.executable, exe, model_dir, "--prompt-ids", "5,9,2", "--max-tokens", "4", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    assert len(json.loads(out.stdout.strip().splitlines()[-1])["tokens"]) == 4
    conf = tmp_path / "c.json"
    conf.write_text(json.dumps(CONFIGS["looped"]))
    out = subprocess.run([sys.executable, exe, "--random", str(conf), "--prompt-len", "9", "--num-prompts", "2",
                          "--max-tokens", "3", "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
