"""The Folivik design on the GPU against its plain implementation.

Each mechanism alone (kernels, and one-layer models whose weights are made so that the key
or the token in question stands out), then whole models in every replay regime, both
precisions, with page pools and state slots so small that everything freed is used again,
the residual stream after every layer, and generation through the engine's own entry point
and scheduler.
"""
import copy
import math

import pytest
import torch

import helpers as H
import folivik_plain as P

pytestmark = pytest.mark.gpu

# largest |difference| / largest |logit|, and rms of the difference / rms of the logits.  The
# float32 bounds are the sharp ones; in bfloat16 every product reads activations rounded to
# eight bits.
TOL = {torch.float32: 6e-5, torch.bfloat16: 0.25}
TOL_RMS = {torch.float32: 1e-5, torch.bfloat16: 6e-2}
F64 = torch.float64


def _runner(model_dir, dtype, page_size, num_pages, max_requests=4):
    from binfer_b200.engine import make_env, make_runner, model_from_dir
    env = make_env(dtype)
    model = model_from_dir(model_dir, env)
    return make_runner(model, env, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests)


def _compare(got, ref, dtype, what, tol_scale=1.0):
    """In bfloat16 a router may decide a close call the other way once its input is rounded,
    which moves that token's logits by more than rounding does: up to two in a hundred
    positions may lie over the bound there (they stay out of the rms too); in float32 none."""
    assert got, "the trace produced no logits"
    worst, worst_at, over = 0.0, None, []
    for (rid, pos), row in got.items():
        e = H.rel_err(row, ref[rid][pos])
        if not e <= TOL[dtype] * tol_scale:
            over.append((rid, pos))
        if not e <= worst:
            worst, worst_at = e, (rid, pos)
    allowed = 0 if dtype == torch.float32 else len(got) // 50
    assert len(over) <= allowed, (f"{what}: {len(over)} of {len(got)} positions over the bound, "
                                  f"worst relative error {worst:.3g} at {worst_at}")
    keep = [k for k in got if k not in set(over)]
    g = torch.stack([got[k] for k in keep])
    r = torch.stack([ref[rid][pos] for (rid, pos) in keep])
    assert H.rel_rms(g, r) <= TOL_RMS[dtype] * tol_scale, f"{what}: rms error {H.rel_rms(g, r):.3g}"
    for rid, lg in ref.items():
        assert all((rid, p) in got for p in range(lg.shape[0])), f"{what}: {rid} incomplete"


def _all_regimes(reqs, tail=10):
    return {"whole": H.trace_whole(reqs), "tail": H.trace_decode_tail(reqs, tail),
            "portions": H.trace_portions(reqs), "mixed": H.trace_mixed(reqs)}


def _one_layer(layer, vocab=260, width=48, eps=1e-5):
    return {"architecture": "Folivik", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [layer]}


SMALL_MOE = H._fol_moe(3, 2, 12, identity=1, groups=(2, 2), scale=1.2, shared=8)


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("off,n", [(0, 24), (7, 50), (16, 1536), (3, 1)])
def test_norm_of_a_column_section(cuda_device, dtype, off, n):
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(n)
    x = (torch.randn(9, off + n + 5, generator=g) * 3).to(dtype)
    w = torch.randn(n, generator=g)
    out = torch.empty(9, n, dtype=dtype, device=cuda_device)
    ops.section_norm(x.to(cuda_device), off, n, w.to(cuda_device), 1e-5, out)
    want = P.rms_norm(x[:, off:off + n].double(), w.double(), 1e-5)
    assert H.rel_err(out.cpu(), want) <= (2e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("n,parts,skip", [(96, 2, True), (40, 5, True), (300, 1, False),
                                          (24, 24, True), (4096, 2, True)])
def test_gate_then_norm_in_parts(cuda_device, n, parts, skip):
    """The gate comes before the norm, and every part has its own root mean square."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(n + parts)
    T = 6
    o = torch.randn(T, n, generator=g)
    sk = torch.randn(T, n, generator=g) if skip else None
    proj = torch.randn(T, n + 7, generator=g)
    w = torch.randn(n, generator=g)
    out = torch.empty(T, n, device=cuda_device)
    ops.gate_norm_out(o.to(cuda_device), sk.to(cuda_device) if skip else None,
                      proj.to(cuda_device), 7, w.to(cuda_device), out, parts, 1e-5)
    y = (o.double() + (sk.double() if skip else 0.0)) * P.silu(proj[:, 7:].double())
    y = y.view(T, parts, n // parts)
    want = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-5)).reshape(T, n) * w.double()
    assert H.rel_err(out.cpu(), want) <= 2e-6
    # the other order (norm, then gate) is another function
    z = o.double() + (sk.double() if skip else 0.0)
    z = z.view(T, parts, n // parts)
    other = ((z / torch.sqrt((z * z).mean(-1, keepdim=True) + 1e-5)).reshape(T, n)
             * w.double() * P.silu(proj[:, 7:].double()))
    if n // parts > 1:
        assert H.rel_err(other, want) > 1e-2


@pytest.mark.parametrize("experts,identity,groups,keep,top,T", [
    (8, 1, 3, 2, 2, 40), (4, 2, 2, 1, 2, 40), (5, 0, 1, 1, 1, 40), (60, 4, 8, 3, 6, 40),
    (2, 2, 2, 2, 4, 40), (16, 0, 4, 4, 4, 700), (30, 3, 33, 5, 5, 40)])
def test_router_over_all_outputs(cuda_device, experts, identity, groups, keep, top, T):
    """Choices and weights against the plain router: corrections that decide choices and lie
    below minus the scores, groups, identity outputs; few and many tokens a launch."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(experts * 10 + identity)
    n, width = experts + identity, 40
    h = torch.randn(T, width, generator=g)
    wr = torch.randn(n, width, generator=g) * 0.4
    corr = torch.randn(n, generator=g) * 0.2 - 0.15
    router = {"experts": experts, "identity": identity, "top": top, "scale": 1.7,
              "groups": {"count": groups, "keep": keep}}
    ids, wts = P.route(h.double(), {"r.router": wr.double(), "r.correction": corr.double()},
                       "r.", router)
    cols = experts + (1 if identity else 0)
    route_w = torch.empty(T, cols, device=cuda_device)
    top_ids = torch.empty(T, top, dtype=torch.int32, device=cuda_device)
    top_w = torch.empty(T, top, device=cuda_device)
    ops.moe_route(h.to(cuda_device), wr.to(cuda_device), experts, top, False, route_w, top_ids,
                  top_w, scoring="softmax_all", correction=corr.to(cuda_device), groups=groups,
                  groups_keep=keep, identity=identity, route_scale=1.7, weight_eps=1e-20)
    want = torch.zeros(T, cols, dtype=F64)
    for t in range(T):
        for e, a in zip(ids[t].tolist(), wts[t].tolist()):
            want[t, min(e, experts)] += a
    # a choice between two nearly equal choice scores may go either way: such tokens aside
    s = torch.softmax(h.double() @ wr.double().T, -1) + corr.double()
    close = torch.zeros(T, dtype=torch.bool)
    for t in range(T):
        v = torch.sort(s[t]).values
        close[t] = bool(((v[1:] - v[:-1]).min() < 1e-6))
    assert int(close.sum()) <= T // 10
    ok = ~close
    assert torch.equal(torch.sort(top_ids.cpu()[ok].long(), -1).values, torch.sort(ids[ok], -1).values)
    assert H.rel_err(route_w.cpu()[ok], want[ok]) <= 2e-6
    assert H.rel_err(top_w.cpu()[ok].sum(-1), wts[ok].sum(-1)) <= 2e-6


def _moe_part(cuda_device, dtype, mlp, width, seed):
    """The feed-forward part built from a configuration's ``mlp`` entry, with random weights,
    and those weights by name."""
    from binfer_b200.config import FolivikConfig
    from binfer_b200.parts.base import BuildEnv, build_ffn
    from binfer_b200.weights import random_tensors
    from binfer_b200.weights.loader import place
    spec = FolivikConfig._mlp(mlp, "mlp.")
    env = BuildEnv(dtype, cuda_device)
    part = build_ffn(spec, width, "f.", env)
    w = random_tensors(part.param_specs(), seed, 0.1, 0.1, dtype)
    w["f.correction"] = (torch.randn(w["f.correction"].shape,
                                     generator=torch.Generator().manual_seed(seed)) * 0.1 - 0.05
                         ).to(dtype)
    by_name = {s.name: s for s in part.param_specs()}
    part.load(lambda s: place(w[s.name], by_name[s.name], dtype, cuda_device))
    return part, w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("mlp,width", [
    (H._fol_moe(8, 2, 32, identity=1, groups=(3, 2), scale=1.5, shared=48), 64),
    (H._fol_moe(4, 3, 16, identity=2, groups=(2, 2), scale=2.5), 48),
    (H._fol_moe(5, 1, 40), 50),
    (H._fol_moe(16, 4, 64, identity=4, groups=(5, 2), scale=1.0, shared=128), 128)])
def test_mixture_of_experts_alone(cuda_device, dtype, mlp, width):
    """The part against the plain mixture: many tokens (every expert is computed) and, in
    bfloat16, one and two tokens (the chosen experts' rows alone are read), with identity
    experts among the choices."""
    part, w = _moe_part(cuda_device, dtype, mlp, width, 5)
    wd = {n: t.double() for n, t in w.items()}
    g = torch.Generator().manual_seed(width)
    chose_identity = 0
    for T in (1, 2, 37):
        h = torch.randn(T, width, generator=g).to(dtype)
        want = P.mixture_of_experts(h.double(), wd, "f.", mlp)
        ids, _ = P.route(h.double(), wd, "f.", mlp["router"])
        chose_identity += int((ids >= mlp["router"]["experts"]).sum())
        got = part.forward(h.to(cuda_device), None)
        assert H.rel_err(got.float().cpu(), want) <= (3e-6 if dtype == torch.float32 else 2e-2), T
    if mlp["router"]["identity"]:
        assert chose_identity > 0


@pytest.mark.parametrize("H_,G_,N,P_", [(4, 2, 16, 24), (3, 3, 8, 8), (2, 1, 40, 12), (2, 1, 6, 10),
                                        (6, 2, 64, 32), (1, 1, 128, 64), (2, 2, 300, 4),
                                        (1, 1, 1, 1), (3, 1, 10, 7), (2, 2, 33, 5)])
def test_scan_with_a_decay_per_token(cuda_device, H_, G_, N, P_):
    """The recurrence alone: unequal requests in one launch, states that continue from slots
    in a shuffled order, against the recurrence written out token by token."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(H_ * 100 + N)
    lens = [70, 1, 17, 2]
    T, B, slots = sum(lens), len(lens), 6
    qk = torch.randn(T, 2, G_, N, generator=g)
    vf = torch.randn(T, H_, P_, generator=g)
    dec = torch.rand(T, H_, generator=g) * 0.5 + 0.5
    dec[:, 0] = 1.0 - 1e-4
    state0 = torch.randn(slots + 1, H_ * N * P_ + 5, generator=g)
    slot_of = [4, 0, 5, 2]
    q_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    state = state0.to(cuda_device)
    o = torch.empty(T, H_ * P_, device=cuda_device)
    err = ops.error_word(cuda_device)
    ops.linear_scan(qk.to(cuda_device), vf.to(cuda_device), dec.to(cuda_device),
                    state[:, :H_ * N * P_], q_start.to(cuda_device),
                    torch.tensor(slot_of, dtype=torch.int32, device=cuda_device), o, B, H_, G_, N,
                    P_, err, max_q=max(lens))
    assert int(err.item()) == 0
    want = torch.zeros(T, H_, P_, dtype=F64)
    end = state0.double().clone()
    for b in range(B):
        for h in range(H_):
            gq = h // (H_ // G_)
            # a slot holds a head's state column by column: [P][N]
            S = state0[slot_of[b], h * N * P_:(h + 1) * N * P_].double().view(P_, N).T.clone()
            for t in range(int(q_start[b]), int(q_start[b + 1])):
                S = dec[t, h].double() * S + torch.outer(qk[t, 1, gq].double(), vf[t, h].double())
                want[t, h] = S.T @ qk[t, 0, gq].double()
            end[slot_of[b], h * N * P_:(h + 1) * N * P_] = S.T.reshape(-1)
    assert H.rel_err(o.cpu(), want.view(T, -1)) <= 3e-6
    assert H.rel_err(state.cpu(), end) <= 3e-6          # untouched slots and columns included


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("heads,groups,state,vdim,conv,parts", [
    (4, 2, 16, 24, 3, 2), (3, 3, 8, 8, 4, 1), (2, 1, 40, 12, 2, 4), (2, 1, 6, 10, 1, 5),
    (1, 1, 128, 64, 4, 1), (6, 3, 72, 20, 5, 3), (2, 2, 320, 6, 2, 2), (3, 1, 10, 7, 3, 3)])
def test_state_space_layer_alone(cuda_device, tmp_path, heads, groups, state, vdim, conv, parts):
    """One layer: a prompt at once, portions, and token by token, over 200 tokens, with a
    decay close to one on the first head, so that the first tokens still count at the end."""
    raw = _one_layer(H._fol_layer("mamba2", H._fol_mamba(heads, groups, state, vdim, conv, parts),
                                  SMALL_MOE))

    def tweak(w):
        w["l0.mix.A_log"][0] = -9.0
        w["l0.mix.dt_bias"][:] += 0.5

    d = H.make_folivik_dir(tmp_path, "A", raw=raw, tweak=tweak, tag=f"m{heads}{state}{vdim}{conv}")
    raw, w = H.read_model_dir(d)
    reqs = {"a": H.random_tokens(200, raw["vocab"], 3), "b": H.random_tokens(37, raw["vocab"], 4)}
    ref = {r: P.forward(raw, w, t) for r, t in reqs.items()}
    other = list(reqs["a"])
    other[2] = (other[2] + 1) % raw["vocab"]
    moved = H.rel_err(P.forward(raw, w, other)[199], ref["a"][199])
    assert moved > 20 * TOL[torch.float32], f"the third token moves the last logits by {moved:.3g} only"
    for name, steps in _all_regimes(reqs, tail=150).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"state space {heads}x{state}x{vdim}/{name}")


def _distinct_tokens(n, vocab, seed):
    return torch.randperm(vocab, generator=torch.Generator().manual_seed(seed))[:n].tolist()


def _mark(w, toks, marked, amp):
    """Two directions of the width are taken out of every embedding; ``e_k`` is put back,
    large, into the embedding of the token at the key's position and ``e_q`` into that of the
    token at the query's (``marked`` = (key, query)).  The layer's first norm passes them, and
    the output head is blind to them, so that the marks themselves add nothing to the logits."""
    gen = torch.Generator().manual_seed(9)
    width, dt = w["embed"].shape[1], w["embed"].dtype
    e_k = torch.randn(width, generator=gen)
    e_k = e_k / e_k.norm()
    e_q = torch.randn(width, generator=gen)
    e_q = e_q - (e_q @ e_k) * e_k
    e_q = e_q / e_q.norm()
    e_k, e_q = e_k.to(dt), e_q.to(dt)
    for e in (e_k, e_q):
        w["embed"] -= torch.outer(w["embed"] @ e, e)
        w["head"] -= torch.outer(w["head"] @ e, e)
    w["embed"][toks[marked[0]]] += e_k * amp
    w["embed"][toks[marked[1]]] += e_q * amp
    w["l0.norm1"].fill_(1.0)
    return e_k, e_q, gen


def _stand_out_window(raw, toks, marked, amp=3.0, boost=4.0):
    """Windowed attention: the first query head of every group answers ``e_q`` with a strong
    fixed vector and the group's key head answers ``e_k`` with the same vector, so that after
    the heads' norms the marked query and the marked key point the same way; that head's
    factor on the scores is raised, so that this one score towers over the others.  The value
    projection is blind to both marks.  (The heads are normed, so a mild boost is enough to
    point a marked head; a large one would only magnify, in every other token, the rounding
    of what is left of the marks' directions.)"""
    mx = raw["layers"][0]["mixer"]
    H_, G_, dk = mx["heads"], mx["kv_heads"], mx["dim"]

    def tweak(w):
        p = "l0.mix."
        e_k, e_q, gen = _mark(w, toks, marked, amp)
        a = torch.randn(dk, generator=gen).to(w["embed"].dtype)
        for g in range(G_):
            h0 = g * (H_ // G_)
            w[p + "q"][h0 * dk:(h0 + 1) * dk] += boost * torch.outer(a, e_q)
            w[p + "k"][g * dk:(g + 1) * dk] += boost * torch.outer(a, e_k)
            w[p + "temp"][h0] = 3.0
        w[p + "q.norm"][:] = 1.0
        w[p + "k.norm"][:] = 1.0
        for e in (e_k, e_q):
            w[p + "v"] -= torch.outer(w[p + "v"] @ e, e)
    return tweak


def _stand_out_latent(raw, toks, marked, amp=3.0, boost=30.0):
    """Latent attention: the down projections write ``e_k`` into the key latent's first number
    and ``e_q`` into the query latent's first number (mildly: the rest of the latents still
    tells tokens apart); the first head's key expansion and query expansion turn those numbers
    into one fixed vector, in the sizes that are not rotated.  That head's values and the
    output projection are made large, so that what the head reads decides the logits."""
    mx = raw["layers"][0]["mixer"]
    d, dv = mx["dim"], mx["vdim"]

    def tweak(w):
        p = "l0.mix."
        e_k, e_q, gen = _mark(w, toks, marked, amp)
        a = torch.randn(d, generator=gen).to(w["embed"].dtype)
        w[p + "dkv"][0] = 0.3 * e_k
        w[p + "dkv.norm"][:] = 1.0
        w[p + "uk"][:d, 0] = a
        w[p + "dq"][0] = 0.3 * e_q
        w[p + "dq.norm"][:] = 1.0
        w[p + "uq"][:d, 0] = boost * a
        w[p + "uv"][:dv] *= 6.0
        w[p + "o"] *= 4.0
    return tweak


# pages of 8: the marked key and the query that asks for it
EDGES = {"far": (3, 230), "first_token": (0, 235), "page_border": (8, 27), "page_end": (7, 24),
         "second_token": (0, 1), "neighbour": (100, 101)}
WINDOW = 24
# (key, query): just inside and just outside a window of 24, in a prompt's part and among
# the tokens decoded alone (the last 100), at a page's first and last place, at the
# sequence's first tokens, and the query's own token
WINDOW_EDGES = {"in_prompt": (77, 100), "out_prompt": (76, 100), "in_decoded": (177, 200),
                "out_decoded": (176, 200), "in_page_start": (8, 31), "out_page_end": (7, 31),
                "first_in": (0, 23), "first_out": (0, 24), "second_out": (1, 25),
                "neighbour": (100, 101), "in_across_the_cut": (130, 150), "out_across_the_cut": (126, 150)}


def _edge_case(cuda_device, tmp_path, raw, tweak_of, key, query, case, wider=None):
    toks = _distinct_tokens(240, raw["vocab"], 21)
    d = H.make_folivik_dir(tmp_path, "A", raw=raw, tweak=tweak_of(raw, toks, (key, query)),
                           tag=case)
    raw, w = H.read_model_dir(d)
    ref = {"a": P.forward(raw, w, toks)}
    if wider is None:
        # the test is only worth something if that one key decides the query's logits: with
        # another token in the key's place they move far beyond the bound
        other = list(toks)
        other[key] = next(t for t in range(raw["vocab"]) if t not in toks)
        moved = H.rel_err(P.forward(raw, w, other)[query], ref["a"][query])
    else:
        # ... or, for a key just outside the window, with a window one token wider
        moved = H.rel_err(P.forward(wider, w, toks)[query], ref["a"][query])
    assert moved > 100 * TOL[torch.float32], f"{case}: the key moves the logits by {moved:.3g} only"
    for name, steps in _all_regimes({"a": toks}, tail=100).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"{case}/{name}")


@pytest.mark.parametrize("case", sorted(WINDOW_EDGES))
def test_windowed_attention_alone_at_its_edges(cuda_device, tmp_path, case):
    """A marked key sits just inside or just outside the window of its query, in prompts, in
    portions and while decoding; where it is outside, a window one token wider would have
    moved the logits."""
    key, query = WINDOW_EDGES[case]
    raw = _one_layer(H._fol_layer("attention", H._fol_attn(4, 2, 16, 24, WINDOW, scale=0.5),
                                  SMALL_MOE), vocab=400)
    wider = None
    if query - key >= WINDOW:
        wider = copy.deepcopy(raw)
        wider["layers"][0]["mixer"]["mask"]["size"] = WINDOW + 1
    _edge_case(cuda_device, tmp_path, raw, _stand_out_window, key, query, case, wider)


@pytest.mark.parametrize("case", sorted(EDGES))
def test_latent_attention_alone_at_its_edges(cuda_device, tmp_path, case):
    """A marked key hundreds of tokens back, at the sequence's start, at a page's border or
    right beside its query, through queries that come out of their own latent."""
    key, query = EDGES[case]
    raw = _one_layer(H._fol_layer("latent_attention",
                                  H._fol_latent(3, 12, 8, 20, 28, 18, scale=0.3), SMALL_MOE),
                     vocab=400)
    _edge_case(cuda_device, tmp_path, raw, _stand_out_latent, key, query, case)


def test_distance_bias_temperature_and_head_norms_count(cuda_device, tmp_path):
    """The plain implementation first shows that leaving out the bias, a head's factor or the
    norms' weights moves the logits; the engine is then held to the full form."""
    raw = _one_layer(H._fol_layer("attention", H._fol_attn(2, 1, 16, 16, 40, scale=0.8)))

    def tweak(w):
        w["l0.mix.r1"][:] = torch.tensor([0.9, 0.4])
        w["l0.mix.r2"][:] = torch.tensor([0.5, 2.0])
        w["l0.mix.temp"][:] = torch.tensor([1.6, 0.7])

    d = H.make_folivik_dir(tmp_path, "A", raw=raw, tweak=tweak, tag="bias")
    raw, w = H.read_model_dir(d)
    toks = H.random_tokens(90, raw["vocab"], 12)
    ref = {"a": P.forward(raw, w, toks)}
    for name, value in (("l0.mix.r1", 0.0), ("l0.mix.temp", 1.0), ("l0.mix.q.norm", 1.0)):
        off = {n: t.clone() for n, t in w.items()}
        off[name][:] = value
        assert H.rel_err(P.forward(raw, off, toks), ref["a"]) > 100 * TOL[torch.float32], name
    for name, steps in _all_regimes({"a": toks}, tail=40).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"bias, factor and norms/{name}")


@pytest.mark.parametrize("heads,d,dr,dv,rank,q_rank,dims", [
    (1, 6, 2, 10, 6, 4, None), (2, 40, 24, 8, 200, 300, None), (5, 8, 40, 30, 12, 16, 20),
    (2, 64, 64, 128, 300, 64, None)])
def test_latent_attention_sizes(cuda_device, tmp_path, heads, d, dr, dv, rank, q_rank, dims):
    """Other sizes: one head, latents smaller and larger than a head, a rotated part larger
    than the plain one and only partly turned, a latent of more than 256 numbers."""
    raw = _one_layer(H._fol_layer("latent_attention",
                                  H._fol_latent(heads, d, dr, dv, rank, q_rank, dims=dims)),
                     width=40)
    dd = H.make_folivik_dir(tmp_path, "B", raw=raw, tag=f"s{heads}{d}{dr}{rank}")
    raw, w = H.read_model_dir(dd)
    reqs = {"a": H.random_tokens(70, raw["vocab"], 5), "b": H.random_tokens(9, raw["vocab"], 6)}
    ref = {r: P.forward(raw, w, t) for r, t in reqs.items()}
    for name, steps in _all_regimes(reqs, tail=30).items():
        got = H.run_trace(_runner(dd, torch.float32, 4, H.peak_pages(steps, 4)), steps)
        _compare(got, ref, torch.float32, f"latent {heads}x{d}+{dr}/{rank}/{name}")


@pytest.mark.parametrize("case", ["in_prompt", "out_prompt", "in_decoded", "out_decoded",
                                  "in_page_start", "out_page_end", "first_out"])
def test_windowed_attention_at_its_edges_on_the_tensor_cores(cuda_device, tmp_path, case):
    """The marked keys again, in bfloat16 and with sizes that the tiled kernel takes (the
    logarithmic bias among them); the profiler shows that it ran.  A model this narrow is
    rounded coarsely in bfloat16 whatever the kernel: the kernel for any sizes on the same
    rounded numbers is the sharp comparison."""
    from binfer_b200.csrc import ops
    from binfer_b200.parts import attention_conv_window as mod
    from binfer_b200.profiling import Profiler
    key, query = WINDOW_EDGES[case]
    raw = _one_layer(H._fol_layer("attention", H._fol_attn(4, 2, 32, 16, WINDOW, scale=0.7),
                                  SMALL_MOE), vocab=400, width=64)
    toks = _distinct_tokens(240, raw["vocab"], 21)
    d = H.make_folivik_dir(tmp_path, "A", torch.bfloat16, raw=raw,
                           tweak=_stand_out_window(raw, toks, (key, query), boost=12.0), tag=case)
    raw, w = H.read_model_dir(d)
    ref = {"a": P.forward(raw, w, toks)}
    if query - key >= WINDOW:
        wider = copy.deepcopy(raw)
        wider["layers"][0]["mixer"]["mask"]["size"] = WINDOW + 1
        moved = H.rel_err(P.forward(wider, w, toks)[query], ref["a"][query])
    else:
        other = list(toks)
        other[key] = next(t for t in range(raw["vocab"]) if t not in toks)
        moved = H.rel_err(P.forward(raw, w, other)[query], ref["a"][query])
    assert moved > 0.3, f"{case}: the key moves the logits by {moved:.3g} only"
    outs = []
    for on in (True, False):
        mod.TENSOR_CORES = on
        seen, got = set(), {}
        try:
            for name, steps in _all_regimes({"a": toks}, tail=100).items():
                prof = Profiler()
                got[name] = H.run_trace(_runner(d, torch.bfloat16, 8, H.peak_pages(steps, 8)), steps)
                prof.stop()
                seen |= set(prof.collect())
                at_query = H.rel_err(got[name][("a", query)], ref["a"][query])
                assert at_query <= 0.25 * moved, (f"{case}/{name} (tensor cores {on}): "
                                                  f"{at_query:.3g} where the key moves {moved:.3g}")
        finally:
            ops.set_profiler(None)
            mod.TENSOR_CORES = True
        assert ("pwm_attention" in seen) == on and ("paged_attention_generic" in seen) != on, sorted(seen)
        outs.append(got)
    for name in outs[0]:
        worst = max(H.rel_err(outs[0][name][k], outs[1][name][k]) for k in outs[0][name])
        assert worst <= 0.03, f"{case}/{name}: the two kernels differ by {worst:.3g}"


@pytest.mark.parametrize("window", [1, 2, 7, 64, 65, 500])
def test_windows_small_and_large_on_the_tensor_cores(cuda_device, tmp_path, window):
    """Windows of one token (a query sees itself alone), of less than a key tile, of exactly a
    tile and one more, and wider than the sequence, in bfloat16 on the tiled kernel and on the
    kernel for any sizes: both within rounding of the plain implementation and of each other."""
    from binfer_b200.parts import attention_conv_window as mod
    raw = _one_layer(H._fol_layer("attention", H._fol_attn(4, 2, 32, 16, window, scale=0.4),
                                  SMALL_MOE), vocab=300, width=64)
    d = H.make_folivik_dir(tmp_path, "D", torch.bfloat16, raw=raw, tag=f"w{window}")
    raw, w = H.read_model_dir(d)
    reqs = {"a": H.random_tokens(150, raw["vocab"], 5), "b": H.random_tokens(66, raw["vocab"], 6)}
    ref = {r: P.forward(raw, w, t) for r, t in reqs.items()}
    if window < 150:
        off = copy.deepcopy(raw)
        off["layers"][0]["mixer"]["mask"]["size"] = window + 1
        assert H.rel_err(P.forward(off, w, reqs["a"]), ref["a"]) > 1e-2
    outs = []
    for on in (True, False):
        mod.TENSOR_CORES = on
        try:
            got = {}
            for name, steps in _all_regimes(reqs, tail=70).items():
                got[name] = H.run_trace(_runner(d, torch.bfloat16, 8, H.peak_pages(steps, 8)), steps)
                _compare(got[name], ref, torch.bfloat16, f"window {window}/{name} (tensor cores {on})")
        finally:
            mod.TENSOR_CORES = True
        outs.append(got)
    for name in outs[0]:
        worst = max(H.rel_err(outs[0][name][k], outs[1][name][k]) for k in outs[0][name])
        assert worst <= 0.05, f"window {window}/{name}: the two kernels differ by {worst:.3g}"


# ----------------------------------------------------------------------- whole models
LENGTHS = {"A": [5, 17, 33, 70, 121], "B": [1, 9, 40, 70, 101], "C": [3, 30, 64, 47, 2],
           "D": [2, 45, 150, 210, 90]}


def _requests(which, extra=()):
    vocab = H.FOL[which]["raw"]["vocab"]
    lens = list(LENGTHS[which]) + list(extra)
    return {f"r{i}": H.random_tokens(n, vocab, 100 * i + n) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def plain_logits(tmp_path_factory):
    cache = {}

    def get(which, dtype, reqs):
        d = H.make_folivik_dir(tmp_path_factory.getbasetemp(), which, dtype)
        raw, w = H.read_model_dir(d)
        out = cache.setdefault((which, dtype), {})
        for rid, toks in reqs.items():
            k = (rid, tuple(toks))
            if k not in out:
                out[k] = P.forward(raw, w, toks)
        return d, {rid: out[(rid, tuple(toks))] for rid, toks in reqs.items()}

    return get


@pytest.mark.parametrize("which,dtype", [("A", torch.float32), ("B", torch.float32),
                                         ("C", torch.float32), ("A", torch.bfloat16),
                                         ("B", torch.bfloat16), ("C", torch.bfloat16),
                                         ("D", torch.bfloat16)],
                         ids=["A-f32", "B-f32", "C-f32", "A-bf16", "B-bf16", "C-bf16", "D-bf16"])
@pytest.mark.parametrize("regime", ["whole", "tail", "portions", "mixed"])
def test_replay(cuda_device, plain_logits, which, dtype, regime):
    """Seven requests through four state slots and page pools of exactly the peak need."""
    reqs = _requests(which, (55, 61) if regime == "mixed" else ())
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = _all_regimes(reqs)[regime]
    ps = H.FOL[which]["page_size"]
    runner = _runner(model_dir, dtype, ps, H.peak_pages(steps, ps))
    got = H.run_trace(runner, steps)
    assert not runner.cache.requests and all(g.pool.num_held == 0 for g in runner.cache.groups)
    assert runner.cache.slots.num_free == 4
    _compare(got, ref, dtype, f"{which}/{regime}")


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_the_stream_after_every_layer(cuda_device, plain_logits, which):
    from binfer_b200.engine.runner import StepItem
    toks = H.random_tokens(19, H.FOL[which]["raw"]["vocab"], 77)
    model_dir, _ = plain_logits(which, torch.float32, {})
    raw, w = H.read_model_dir(model_dir)
    want = []
    P.forward(raw, w, toks, want)
    runner = _runner(model_dir, torch.float32, 8, 4)
    runner.add_request("a")
    items = [StepItem("a", toks, [len(toks) - 1])]
    runner.reserve(items)
    runner.cache.zero_fresh_state(runner.cache.get("a"))
    ctx = runner.build_context(items)
    ctx.scratch["layer_outputs"] = []
    runner.model.forward(ctx, runner.views)
    got = ctx.scratch["layer_outputs"]
    assert len(got) == len(want) == len(runner.model.spec.schedule)
    for i, (g, r) in enumerate(zip(got, want)):
        assert H.rel_err(g.cpu(), r) <= 2e-5, f"{which}: after layer {i}"


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_regimes_agree_bitwise_in_float32(cuda_device, plain_logits, which):
    """Every sum's order depends on positions and sizes alone: cutting and batching change
    no bit."""
    reqs = _requests(which)
    model_dir, _ = plain_logits(which, torch.float32, reqs)
    ps = H.FOL[which]["page_size"]
    outs = []
    for steps in _all_regimes(reqs).values():
        outs.append(H.run_trace(_runner(model_dir, torch.float32, ps, H.peak_pages(steps, ps)),
                                steps))
    for other in outs[1:]:
        for key, row in outs[0].items():
            assert torch.equal(row, other[key]), f"{which}: logits at {key} depend on the cut"


def test_long_decoding(cuda_device, plain_logits):
    """A short prompt, then 300 tokens one by one: the window passes over decoded tokens and
    the recurrent state is carried 300 times."""
    which, dtype = "B", torch.float32
    reqs = {"long": H.random_tokens(304, H.FOL[which]["raw"]["vocab"], 7)}
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_decode_tail(reqs, tail=300)
    runner = _runner(model_dir, dtype, 4, 76)
    _compare(H.run_trace(runner, steps), ref, dtype, "long decoding")


def test_decoding_from_captured_steps(cuda_device, plain_logits):
    """Steps of single tokens replayed from CUDA graphs (padded rows use the scratch page and
    the scratch state slot) give what eager steps give."""
    which, dtype = "A", torch.float32
    reqs = _requests(which, (55, 61))
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_mixed(reqs, tail=20)
    ps = H.FOL[which]["page_size"]
    runner = _runner(model_dir, dtype, ps, H.peak_pages(steps, ps))
    runner.enable_decode_graphs(max_batch=4, max_seq_len=256)
    got = H.run_trace(runner, steps)
    assert getattr(runner, "graph_replays", 0) > 0
    _compare(got, ref, dtype, "captured decode steps")


# ------------------------------------------------------------------------- generation
@pytest.mark.parametrize("graphs,step_tokens", [(True, 2048), (False, 7)],
                         ids=["graphs", "portions"])
def test_greedy_generation_through_the_engine(cuda_device, tmp_path, graphs, step_tokens):
    """Prompts of 5/17/33/2 tokens through ``Engine.generate``: the scheduler's admission,
    portions of at most seven tokens beside decoding (second case), captured decode steps
    (first case); every token is the plain implementation's choice."""
    from binfer_b200 import Engine
    d = H.make_folivik_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab"], n) for n in (5, 17, 33, 2)]
    eng = Engine(d, "float32", num_pages=40, page_size=16, max_seq_len=128, max_batch_size=3,
                 max_tokens_per_step=step_tokens, cuda_graphs=graphs)
    got = eng.generate(prompts, max_tokens=12, ignore_eos=True)
    for p, out in zip(prompts, got):
        assert len(out) == 12
        logits = P.forward(raw, w, list(p) + list(out))
        for n, tok in enumerate(out):
            row = logits[len(p) - 1 + n]
            assert float(row[tok]) >= float(row.max()) - 1e-4 * float(row.abs().max()), (
                f"token {n} after a prompt of {len(p)}: {tok}, plain {int(row.argmax())}")
    st = eng.stats()
    assert st["pages_free"] == st["pages_total"]
    if graphs:
        assert getattr(eng.runner, "graph_replays", 0) > 0


def test_command_line_generates_from_a_folder(cuda_device, tmp_path, capsys):
    """``bin/binfer``'s entry point: the registry picks the family from config.json; greedy
    tokens are the plain implementation's, and sampling with a seed gives the same tokens
    twice."""
    from binfer_b200.cli import main
    d = H.make_folivik_dir(tmp_path, "C")
    raw, w = H.read_model_dir(d)
    prompt = H.random_tokens(9, raw["vocab"], 3)
    ids = ",".join(map(str, prompt))
    rc = main([d, "--prompt-ids", ids, "--max-tokens", "5", "--dtype", "fp32", "--ignore-eos",
               "-q", "--kv-pages", "32"])
    assert rc == 0
    out = [int(t) for t in capsys.readouterr().out.split()]
    assert len(out) == 5
    logits = P.forward(raw, w, list(prompt) + out)
    for n, tok in enumerate(out):
        row = logits[len(prompt) - 1 + n]
        assert float(row[tok]) >= float(row.max()) - 1e-4 * float(row.abs().max())
    sampled = []
    for _ in range(2):
        rc = main([d, "--prompt-ids", ids, "--max-tokens", "8", "--dtype", "fp32", "--ignore-eos",
                   "-q", "--kv-pages", "32", "--temperature", "0.9", "--seed", "5"])
        assert rc == 0
        sampled.append(capsys.readouterr().out.split())
    assert sampled[0] == sampled[1] and len(sampled[0]) == 8


def test_trace_replay_tool_with_four_state_slots(cuda_device, tmp_path):
    """``bin/trace_run`` as a user runs it: six requests through its four state slots and a
    page pool sized by ``--max-tokens``."""
    import test_trace_run_gpu as TR
    d = H.make_folivik_dir(tmp_path, "B")
    raw, w = H.read_model_dir(d)
    reqs = {f"r{i}": H.random_tokens(n, raw["vocab"], 31 * i + n)
            for i, n in enumerate([70, 33, 90, 12, 64, 41])}
    steps = H.trace_mixed(reqs)
    live, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values()))
        for rid in st["end"]:
            live.pop(rid)
    out_dir = str(tmp_path / "out")
    TR._replay(d, "float32", steps, out_dir, peak)
    got = TR._collect(steps, out_dir, raw["vocab"])
    ref = {rid: P.forward(raw, w, toks) for rid, toks in reqs.items()}
    worst = max(H.rel_err(row, ref[rid][p]) for (rid, p), row in got.items())
    assert got and worst <= TOL[torch.float32], f"worst relative error {worst:.3g}"
