"""Pepolorn on the device against the plain implementation in ``plain_pepolorn.py``: every mechanism alone, then
whole models of several shapes through the replay session (whole prompts, decoding token by token, portions down
to two tokens, mixed batches with pages and state slots used again) and greedy generation through the engine and
its scheduler."""
import json
import os

import numpy as np
import pytest
import torch

import plain_pepolorn as P
import replay_util as U

pytestmark = pytest.mark.gpu


def _ssm(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def _par(left, right, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def _att(heads, kv_heads, dim, vdim, chunk, dims, base=10000.0, scale=None, scaling=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5 * 2.0,
            "mask": {"size": chunk}, "rot": {"base": base, "dims": dims, "scaling": scaling}}


def _lin(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def _moe(experts, top, count, keep, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}},
            "expert": {"ff": ff}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _cfg(layers, width=48, vocab=101, eps=1e-5):
    return {"architecture": "Pepolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def _with(layer, mlp, **more):
    return dict(layer, mlp=mlp, **more)


YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
_PAR_A = _par(_att(3, 1, 32, 16, 37, 8, base=300.0, scale=0.35, scaling=YARN), _lin(2, 16, 24, [0.7, 0.97]), 1.3, 0.4)
CONFIGS = {
    # both kinds of mixer, value heads shorter than key heads, part of a head rotated with rescaled frequencies, a
    # chunk that is no multiple of a page, a layer that runs another layer's tensors, a layer without feed-forward
    "both_mixers": _cfg([_with(_ssm(6, 8, 16, groups=3, conv=4, norm_groups=2), _dense(72)),
                         _with(_PAR_A, _moe(6, 2, 3, 2, 24)),
                         _with(_ssm(2, 16, 32, conv=3), None),
                         _with(_PAR_A, _moe(6, 2, 3, 2, 24), weights_of=1)]),
    # the values a model may happen to make equal or one: as many kv heads as heads, one group everywhere, the whole
    # head rotated without rescaling, two taps, one expert a token, scales of one, value heads longer than key heads
    "equal_or_one": _cfg([_with(_par(_att(2, 2, 16, 32, 16, 16, base=50.0), _lin(1, 32, 32, [0.9]), 1.0, 1.0), _moe(4, 1, 1, 1, 32)),
                          _with(_ssm(1, 32, 16, groups=1, conv=2, norm_groups=1), _dense(64)),
                          _with(_ssm(1, 32, 16, groups=1, conv=2, norm_groups=1), _dense(64), weights_of=1)], width=64, vocab=131),
    # sizes that no fast path takes: a width that is no multiple of 8, heads of 40 and 12, a state of 20, five taps,
    # nine experts in three open groups, a chunk of one page
    "odd_sizes": _cfg([_with(_ssm(3, 12, 20, groups=1, conv=5, norm_groups=3), _moe(9, 4, 3, 3, 20)),
                       _with(_par(_att(4, 2, 40, 40, 8, 12, base=77.0, scaling={"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}),
                                  _lin(3, 12, 20, [0.5, 0.8, 0.999]), 0.8, 1.7), _dense(50))], width=36, vocab=50),
    # recurrent layers only: no pages at all, only state slots
    "recurrent_only": _cfg([_with(_ssm(4, 8, 8, groups=2, conv=3, norm_groups=2), _moe(4, 2, 2, 1, 16)),
                            _with(_ssm(2, 24, 48, groups=2, conv=4, norm_groups=1), None)], width=40),
}


def _model_dir(tmp_path, name, cfg, seed=1, static_choice=False, edit=None):
    """``static_choice``: the corrections are spread so widely (steps of 1.5, scores lie in (0, 1)) that they alone
    decide which experts are chosen.  Whole models in bfloat16 use it: a choice that flips by rounding changes a
    row by much more than rounding, and the recurrent layers behind it carry the change to every later row.  The
    weights stay the plain scores, so the experts' products and the weighted sum are still held to the plain ones."""
    w = P.random_weights(cfg, seed)
    if static_choice:
        g = torch.Generator().manual_seed(seed)
        for k in w:
            if k.endswith(".correction"):
                w[k] = 1.5 * torch.randperm(w[k].numel(), generator=g).double()
    if edit is not None:
        edit(w)
    U.write_model_dir(str(tmp_path / name), cfg, {k: v.float() for k, v in w.items()}, torch.bfloat16)
    return str(tmp_path / name), w


def _session(model_dir, dtype, max_tokens, block=16, max_requests=4):
    from firefly_b200.replay import ReplaySession
    return ReplaySession(model_dir, dtype=dtype, max_tokens=max_tokens, block_size=block, max_requests=max_requests)


def _compare_most(got, plain, tol, what, frac=0.9):
    """``frac`` of the rows within tol, and every row finite and within 1.  The norm on a part's output divides by
    that output's root mean square: a row whose part happens to give a small output has its bfloat16 rounding
    magnified, and the recurrent layers behind it carry that to the sequence's later rows (the 32-bit runs of the
    same schedules hold every row)."""
    errs = sorted(U.rel_err(row, plain[rid.split("#")[0]][pos]) for (rid, pos), row in got.rows.items())
    assert errs and all(e == e for e in errs), what
    assert errs[-1] <= 1.0 and errs[int(frac * (len(errs) - 1))] <= tol, \
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
    model_dir, w = _model_dir(tmp_path, name, cfg, static_choice=dtype == "bfloat16")
    reqs = U.make_requests(cfg["vocab"], [70, 3, 45, 1, 33, 58], 5)
    plain = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    twice = dict(reqs, **{"r0#2": reqs["r0"], "r4#2": reqs["r4"]})       # a request once more, on pages and slots used before
    for label, steps in (("whole", U.trace_whole(reqs)), ("decode", U.trace_tail_decode(reqs, tail=40)),
                         ("portions", U.trace_portions(reqs, sizes=(17, 5, 2, 9, 2, 31, 3, 2))),
                         ("mixed", U.trace_mixed(twice, seed=3, max_live=4, sizes=(13, 2, 7, 21, 3, 2, 16)))):
        sess = _session(model_dir, dtype, U.peak_tokens(steps), block=16 if label != "portions" else 8)
        got = U.run_trace(sess, steps)
        _check(got, plain, dtype, f"{name}/{dtype}/{label}")
        sess.cache.check()
        assert not sess.cache.live


def test_the_stream_matches_after_every_layer(tmp_path):
    cfg = CONFIGS["both_mixers"]
    model_dir, w = _model_dir(tmp_path, "stream", cfg)
    toks = U.make_requests(cfg["vocab"], [45], 8)["r0"]
    want = []
    P.forward(cfg, w, toks, want)
    sess = _session(model_dir, "float32", 64)
    got = []
    sess.model.after_run = lambda i, res, pending: got.append(res.detach().cpu().double().clone())
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": ["a"]})
    assert len(got) == len(cfg["layers"]) == 4
    for i, g in enumerate(got):
        assert float((g - want[i]).abs().max()) < 2e-5 * float(want[i].abs().max()), f"after layer {i}"


# ------------------------------------------------------------------ mechanisms alone --
def _one_layer(tmp_path, layer, width=48, dtype="float32", seed=2, max_tokens=1024, block=16, edit=None):
    cfg = _cfg([layer], width=width)
    model_dir, w = _model_dir(tmp_path, "one", cfg, seed, edit=edit)
    return cfg, w, _session(model_dir, dtype, max_tokens, block=block)


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


def _run_cut(sess, mixer, x, cuts, rid):
    rows, p = [], 0
    for n in cuts:
        ctx, entries = _step_context(sess, [(rid, n)])
        out = mixer.forward(x[p:p + n].cuda().contiguous(), ctx, 0, True)
        rows.append(out.float().cpu())
        _advance(sess, entries)
        p += n
    sess.cache.free(sess.live.pop(rid))        # pages and slot go to the next cutting, which must start from zero
    return torch.cat(rows).double()


CUTS = ([57], [20, 2, 1, 1, 30, 3], [1] * 57)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(6, 8, 16, 3, 4, 2), (1, 40, 24, 1, 2, 1), (2, 128, 128, 2, 1, 4), (2, 4, 100, 1, 3, 1), (3, 64, 128, 1, 6, 3),
                                   (1, 160, 200, 1, 2, 1)])
def test_state_space_mixer_alone_whole_in_portions_and_token_by_token(tmp_path, dtype, shape):
    heads, vdim, state, groups, conv, parts = shape
    layer = _with(_ssm(heads, vdim, state, groups, conv, parts), None)
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    x = torch.randn(57, 48, generator=torch.Generator().manual_seed(0)).to(tdt)
    want = P.mamba2_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"])
    mixer = sess.model.blocks[0].mixer
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in CUTS:
        got = _run_cut(sess, mixer, x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 16, 24, [0.7, 0.97]), (1, 128, 128, [0.999]), (3, 12, 20, [0.5, 1.0, 0.9]), (1, 192, 256, [0.9])])
def test_linear_attention_alone_whole_in_portions_and_token_by_token(tmp_path, dtype, shape):
    heads, dim, vdim, decay = shape
    layer = _with(_par(_att(1, 1, 16, 16, 8, 16), _lin(heads, dim, vdim, decay)), None)
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    x = torch.randn(57, 48, generator=torch.Generator().manual_seed(1)).to(tdt)
    want, _ = P.lightning_attention(x.double(), w, "l0.mix.right", layer["mixer"]["right"], cfg["norm"]["eps"])
    mixer = sess.model.blocks[0].mixer.mixers[1]
    from firefly_b200.cache.spec import sub_slot
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in CUTS:
        rid, rows, p = f"r{len(cuts)}", [], 0
        for n in cuts:
            ctx, entries = _step_context(sess, [(rid, n)])
            rows.append(mixer.forward(x[p:p + n].cuda().contiguous(), ctx, sub_slot(0, 1), True).float().cpu())
            _advance(sess, entries)
            p += n
        sess.cache.free(sess.live.pop(rid))
        got = torch.cat(rows).double()
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts


def test_recurrent_state_of_a_freed_slot_does_not_leak_and_batches_equal_requests_alone(tmp_path):
    layer = _with(_ssm(4, 8, 16, 2, 4, 2), None)
    cfg, w, sess = _one_layer(tmp_path, layer)
    g = torch.Generator().manual_seed(1)
    xs = {rid: torch.randn(n, 48, generator=g) * 2 for rid, n in (("a", 9), ("b", 1), ("c", 30), ("d", 2))}
    want = {rid: P.mamba2_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"]) for rid, x in xs.items()}
    mixer = sess.model.blocks[0].mixer
    for rounds in range(2):                       # the second round runs on slots the first one used
        ctx, entries = _step_context(sess, [(rid, x.shape[0]) for rid, x in xs.items()])
        order = [e.cache.request_id for e in sorted(entries, key=lambda e: 0 if len(e.tokens) == 1 else 1)]
        got = mixer.forward(torch.cat([xs[r] for r in order]).cuda(), ctx, 0, True).cpu().double()
        p = 0
        for r in order:
            n = xs[r].shape[0]
            assert float((got[p:p + n] - want[r]).abs().max()) < 3e-5 * float(want[r].abs().max()), (rounds, r)
            p += n
        for rid in xs:
            sess.cache.free(sess.live.pop(rid))


def _queries_like_keys(w, p, att):
    """Every query head gets minus the matrix of the key head it reads: a row that is minus an earlier row then
    has, in the unrotated part of the head, a query along that row's key (and against its own), and with
    unit-normed q and k that one score stands far above the others.  An attention that loses or wrongly sees that
    key gives another result."""
    d = att["dim"]
    for h in range(att["heads"]):
        kh = h // (att["heads"] // att["kv_heads"])
        w[p + ".q"][h * d:(h + 1) * d] = -w[p + ".k"][kh * d:(kh + 1) * d]


def _standout_inputs(T, width, far, query, seed):
    x = torch.randn(T, width, generator=torch.Generator().manual_seed(seed)) * 0.5
    x[query] = -x[far]
    return x


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk,far,query", [(64, 64, 120), (64, 63, 120), (64, 0, 63), (64, 128, 129), (64, 127, 128),
                                            (40, 80, 119), (40, 79, 119), (200, 200, 419), (200, 199, 419), (16, 15, 16)])
def test_chunked_attention_alone_sees_its_chunk_and_nothing_else(tmp_path, dtype, chunk, far, query):
    """A key that stands out, just inside or just outside the query's chunk, at and off page borders, with the
    query inside a prompt's portion, at the start of a portion, and decoded alone."""
    att = _att(4, 2, 24, 24, chunk, 4, base=100.0, scale=1.5)
    layer = _with(_par(att, _lin(1, 8, 8, [0.5]), 1.0, 0.0), None)       # the other mixer's share is switched off
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype, edit=lambda w: _queries_like_keys(w, "l0.mix.left", att))
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    T = query + 1
    x = _standout_inputs(T, 48, far, query, far).to(tdt)
    want = P.chunked_attention(x.double(), w, "l0.mix.left", att, cfg["norm"]["eps"])
    # the test can tell: with every key visible (one chunk) the query row changes exactly when `far` is outside
    every = P.chunked_attention(x.double(), w, "l0.mix.left", dict(att, mask={"size": 1 << 20}), cfg["norm"]["eps"])
    inside = far // chunk == query // chunk
    moved = float((every[-1] - want[-1]).abs().max()) > 0.1 * float(want[-1].abs().max())
    assert moved == (not inside)
    if inside:
        other = x.clone()
        other[far] = other[far - 1] if far else other[far + 1]
        lost = P.chunked_attention(other.double(), w, "l0.mix.left", att, cfg["norm"]["eps"])
        assert float((lost[-1] - want[-1]).abs().max()) > 0.1 * float(want[-1].abs().max())
    mixer = sess.model.blocks[0].mixer
    tol = 3e-5 if dtype == "float32" else 4e-2
    cuttings = [[T], [T - 1, 1], [far + 1, T - far - 1]] + ([[far, T - far - 2, 2]] if T - far > 2 and far else [])
    for cuts in cuttings:
        got = _run_cut(sess, mixer, x, [c for c in cuts if c], f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts
        assert float((got[-1] - want[-1]).abs().max()) <= tol * float(want[-1].abs().max()), cuts


def test_parallel_mixers_in_a_batch_of_unequal_requests_on_reused_pages_and_slots(tmp_path):
    layer = _with(_PAR_A, None)
    cfg, w, sess = _one_layer(tmp_path, layer, max_tokens=512, block=8)
    g = torch.Generator().manual_seed(4)
    mixer = sess.model.blocks[0].mixer
    for rounds in range(3):
        xs = {rid: torch.randn(n, 48, generator=g) for rid, n in (("a", 70), ("b", 1), ("c", 129), ("d", 2))}
        want = {rid: P.parallel_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"]) for rid, x in xs.items()}
        done = {rid: 0 for rid in xs}
        for take in ({"a": 33, "b": 1, "c": 64, "d": 1}, {"a": 36, "c": 1, "d": 1}, {"a": 1, "c": 64}):
            ctx, entries = _step_context(sess, list(take.items()))
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


@pytest.mark.parametrize("dims,scaling", [(8, None), (24, YARN), (2, {"factor": 3.0, "original": 16, "fast": 2.0, "slow": 0.5})])
def test_rotation_then_unit_norm_alone(dims, scaling):
    from types import SimpleNamespace
    from firefly_b200.ops import kernels as K
    from firefly_b200.config.base import PartSpec
    from firefly_b200.parts import Runtime, build_part
    rot = {"base": 123.0, "dims": dims, "scaling": scaling}
    pos_part = build_part("position", PartSpec("rotary", dict(head_dim=24, rotary_dim=dims, theta=123.0, max_positions=0,
                                                               scaling=scaling)), Runtime(torch.device("cuda"), torch.float32))
    f, mag = P.rotary_frequencies(rot)
    assert torch.allclose(pos_part.frequencies().cpu(), f, rtol=1e-14) and abs(pos_part.magnitude - mag) < 1e-15
    positions = torch.tensor([0, 1, 7, 1000, 123456], dtype=torch.int32)
    q = torch.randn(5, 3 * 24, generator=torch.Generator().manual_seed(dims))
    want = P.rms(P.rotate(q.double().view(5, 3, 24), positions, rot), 1e-5).reshape(5, 72)
    ctx = SimpleNamespace(positions=positions.cuda(), token_seq=torch.zeros(5, dtype=torch.int32, device="cuda"),
                          status=torch.zeros(1, dtype=torch.int32, device="cuda"))
    got = q.cuda()
    K.rope_unit_norm_store(got, 3, 0, 24, 24, 1e-5, pos_part.frequencies(), pos_part.magnitude, ctx, None, None)
    assert float((got.cpu().double() - want).abs().max()) < 2e-6


@pytest.mark.parametrize("shape", [(6, 2, 3, 2), (8, 3, 8, 4), (4, 1, 1, 1), (12, 4, 2, 1), (5, 5, 1, 1), (12, 2, 3, 2), (9, 3, 9, 3)])
def test_router_choice_and_weights(shape):
    from firefly_b200.ops import kernels as K
    E, top, count, keep = shape
    g = torch.Generator().manual_seed(E * 7 + top)
    h = torch.randn(64, 16, generator=g).double()
    # corrections large enough to change the choice, negative enough that choice scores fall below zero
    w = {"r.router": torch.randn(E, 16, generator=g).double(), "r.correction": torch.randn(E, generator=g).double() - 0.8}
    r = {"experts": E, "top": top, "groups": {"count": count, "keep": keep}}
    want_ids, want_w = P.route(h, w, "r", r)
    assert float((torch.sigmoid(h @ w["r.router"].T) + w["r.correction"]).min()) < 0
    z = (h @ w["r.router"].T).float().cuda()
    ids = torch.empty(64, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(64, top, dtype=torch.float32, device="cuda")
    K.moe_route(z, ids, wts, count, keep, score=K.ROUTE_SIGMOID, correction=w["r.correction"].float().cuda(),
                group_score=K.GROUP_BY_TWO_BEST, renormalize=False)
    assert ids.cpu().tolist() == want_ids.tolist()
    assert torch.allclose(wts.cpu().double(), want_w, rtol=1e-5, atol=1e-7)
    # a choice without the correction differs somewhere: the test can tell that it is used
    K.moe_route(z, ids, wts, count, keep, score=K.ROUTE_SIGMOID, group_score=K.GROUP_BY_TWO_BEST, renormalize=False)
    if top < E:
        assert ids.cpu().tolist() != want_ids.tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens", [1, 5, 150])
def test_feed_forwards_alone(tmp_path, dtype, tokens):
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(tokens)
    x = (torch.randn(tokens, 48, generator=g) * 1.5).to(tdt)
    for mlp in (_moe(6, 2, 3, 2, 24), _dense(72)):
        cfg, w, sess = _one_layer(tmp_path, _with(_ssm(1, 8, 8), mlp), dtype=dtype)
        want = P.moe_ff(x.double(), w, "l0.mlp", mlp) if mlp["kind"] == "moe" else P.dense_ff(x.double(), w, "l0.mlp")
        ctx, _ = _step_context(sess, [("a", tokens)])
        ff = sess.model.blocks[0].feed_forward
        delta = torch.zeros(tokens, 48, device="cuda")
        left = ff.forward(x.cuda(), ctx, accumulate_into=delta)
        got = (delta if left is None else left).float().cpu().double()
        err = (got - want).abs().max(dim=1).values / want.abs().max()
        if dtype == "float32":
            assert float(err.max()) < 2e-5, mlp["kind"]
        else:
            assert float(err.sort().values[int(0.95 * (tokens - 1))]) < 3e-2, mlp["kind"]


def test_the_recurrence_kernels_layout_is_the_one_the_host_sizes_state_slots_for():
    from firefly_b200.ops import kernels as K
    for N in (1, 8, 16, 17, 32, 33, 64, 65, 100, 128, 129, 256):
        for V in (1, 8, 12, 31, 32, 33, 64, 100, 128, 130, 256):
            assert K.scan_state_floats(3, N, V) == K.scan_state_floats_of_kernel(3, N, V), (N, V)


@pytest.mark.parametrize("H", [40, 37, 4100, 16388])
def test_norm_on_a_parts_output_alone(H):
    from firefly_b200.ops import kernels as K
    g = torch.Generator().manual_seed(3)
    res, delta, w = torch.randn(11, H, generator=g) * 3, torch.randn(11, H, generator=g) * 5, torch.randn(H, generator=g) * 0.1
    want = res.double() + P.offset_norm(delta.double(), w.double(), 1e-5)
    for dt in (torch.float32, torch.bfloat16):
        r, copy = res.cuda(), torch.empty(11, H, dtype=dt, device="cuda")
        d = delta.to(dt)
        K.norm_add(r, d.cuda(), (1.0 + w).cuda(), 1e-5, copy)
        ref = res.double() + P.offset_norm(d.double(), w.double(), 1e-5)
        assert float((r.cpu().double() - ref).abs().max()) < 1e-5
        assert torch.equal(copy.cpu(), r.cpu().to(dt))
    assert float((ref - want).abs().max()) < 0.2


# ------------------------------------------------------------------ long decoding, generation --
def test_long_decoding_keeps_state_and_cache(tmp_path):
    cfg = CONFIGS["both_mixers"]
    model_dir, w = _model_dir(tmp_path, "long", cfg, seed=4)
    toks = U.make_requests(cfg["vocab"], [200], 2)["r0"]
    plain = {"r0": P.forward(cfg, w, toks).numpy()}
    steps = U.trace_tail_decode({"r0": toks}, tail=190)          # the chunk's edge passes five times while decoding
    sess = _session(model_dir, "float32", U.peak_tokens(steps), block=8)
    U.compare(U.run_trace(sess, steps), plain, U.TOL["float32"], "long decoding")


def test_the_first_tokens_of_a_sequence(tmp_path):
    cfg = CONFIGS["odd_sizes"]
    model_dir, w = _model_dir(tmp_path, "first", cfg, seed=5)
    reqs = U.make_requests(cfg["vocab"], [1, 2, 3, 6], 9)
    plain = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    for steps in (U.trace_whole(reqs), U.trace_tail_decode(reqs, tail=5), U.trace_portions(reqs, sizes=(2, 1, 3))):
        sess = _session(model_dir, "float32", 256)
        U.compare(U.run_trace(sess, steps), plain, U.TOL["float32"], "first tokens")


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path, graphs, dtype):
    from firefly_b200 import LLM
    cfg = CONFIGS["both_mixers"]
    model_dir, w = _model_dir(tmp_path, "gen", cfg, seed=6, static_choice=dtype == "bfloat16")
    prompts = [v for v in U.make_requests(cfg["vocab"], [19, 3, 41, 8, 27], 11).values()]
    llm = LLM(model_dir, dtype=dtype, max_batch_size_limit=3, kv_block_size=8, num_kv_blocks=40,
              max_prefill_chunk_size=16, eos_token_ids=[], use_cuda_graphs=graphs)
    outs = llm.generate(prompts, max_tokens=10, ignore_eos=True)
    llm.engine.cache.check()
    close = 1e-4 if dtype == "float32" else 5e-2
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        rows = P.forward(cfg, w, list(p) + o[:-1])
        for i, tok in enumerate(o):
            row = rows[len(p) - 1 + i]
            top2 = torch.topk(row, 2).values
            assert tok == int(row.argmax()) or float(row.max() - row[tok]) < close * float(row.abs().max()), (i, tok)


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
    conf.write_text(json.dumps(CONFIGS["both_mixers"]))
    out = subprocess.run([sys.executable, exe, "--random", str(conf), "--prompt-len", "9", "--num-prompts", "2",
                          "--max-tokens", "3", "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
