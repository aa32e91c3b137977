"""The looped design on the GPU against its plain implementation.

Each mechanism alone (kernels, and one-layer models whose weights are made so that the key
in question stands out), then whole models in every replay regime, both precisions, with
page pools and state slots so small that everything freed is used again, the residual
stream after every layer run, and generation through the engine's own entry point and
scheduler.
"""
import copy

import pytest
import torch

import helpers as H
import ketopel_plain as P

pytestmark = pytest.mark.gpu

# largest |difference| / largest |logit|, and rms of the difference / rms of the logits.  The
# float32 bounds are the sharp ones; in bfloat16 every product reads activations rounded to
# eight bits.
TOL = {torch.float32: 6e-5, torch.bfloat16: 0.25}
TOL_RMS = {torch.float32: 1e-5, torch.bfloat16: 6e-2}


def _runner(model_dir, dtype, page_size, num_pages, max_requests=4):
    from binfer_b200.engine import make_env, make_runner, model_from_dir
    env = make_env(dtype)
    model = model_from_dir(model_dir, env)
    return make_runner(model, env, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests)


def _compare(got, ref, dtype, what, tol_scale=1.0):
    assert got, "the trace produced no logits"
    worst, worst_at = 0.0, None
    for (rid, pos), row in got.items():
        e = H.rel_err(row, ref[rid][pos])
        if not e <= worst:
            worst, worst_at = e, (rid, pos)
    assert worst <= TOL[dtype] * tol_scale, (f"{what}: worst relative error {worst:.3g} at "
                                            f"{worst_at}")
    keys = list(got)
    g = torch.stack([got[k] for k in keys])
    r = torch.stack([ref[rid][pos] for (rid, pos) in keys])
    assert H.rel_rms(g, r) <= TOL_RMS[dtype] * tol_scale, f"{what}: rms error {H.rel_rms(g, r):.3g}"
    for rid, lg in ref.items():
        assert all((rid, p) in got for p in range(lg.shape[0])), f"{what}: {rid} incomplete"


def _all_regimes(reqs, tail=10):
    return {"whole": H.trace_whole(reqs), "tail": H.trace_decode_tail(reqs, tail),
            "portions": H.trace_portions(reqs), "mixed": H.trace_mixed(reqs)}


def _one_layer(layer, vocab=260, width=48, eps=1e-5, scale=1.5, loop=None):
    raw = {"architecture": "Ketopel", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "layers": [layer]}
    if loop:
        raw["loop"] = loop
    return raw


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("inner", [24, 50, 257, 1024])
def test_gated_activation_in_gelu_tanh_form(cuda_device, dtype, inner):
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(inner)
    gu = (torch.randn(9, 2 * inner, generator=g) * 3).to(dtype)
    out = torch.empty(9, inner, dtype=dtype, device=cuda_device)
    ops.gated_act_mul(gu.to(cuda_device), out, "gelu_tanh")
    want = P.gelu_tanh(gu[:, :inner].double()) * gu[:, inner:].double()
    assert H.rel_err(out.cpu(), want) <= (2e-6 if dtype == torch.float32 else 6e-3)
    ops.gated_act_mul(gu.to(cuda_device), out, "silu")
    want = P.silu(gu[:, :inner].double()) * gu[:, inner:].double()
    assert H.rel_err(out.cpu(), want) <= (2e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_what_a_pass_starts_with(cuda_device, dtype):
    """The stream takes its pending sublayer output, the embedding output again and a row of
    the pass table in one kernel; each of the three may be absent."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    T, width, vocab = 11, 70, 40
    x = torch.randn(T, width, generator=g)
    delta = torch.randn(T, width, generator=g).to(dtype)
    table = torch.randn(vocab, width, generator=g).to(dtype)
    vec = torch.randn(width, generator=g)
    ids = torch.randint(0, vocab, (T,), generator=g, dtype=torch.int32)
    err = ops.error_word(cuda_device)
    for use in ((1, 1, 1), (0, 1, 1), (1, 0, 1), (0, 0, 1), (1, 1, 0)):
        resid = x.to(cuda_device)
        ops.stream_inject(resid, delta.to(cuda_device) if use[0] else None,
                          table.to(cuda_device) if use[1] else None, ids.to(cuda_device), 2.5,
                          vec.to(cuda_device) if use[2] else None, err)
        want = x.double()
        if use[0]:
            want = want + delta.double()
        if use[1]:
            want = want + table.double()[ids.long()] * 2.5
        if use[2]:
            want = want + vec.double()
        assert H.rel_err(resid.cpu(), want) <= 1e-6
    assert int(err.item()) == 0


@pytest.mark.parametrize("heads,dv,over_all,shared", [(3, 20, True, False), (2, 48, False, True),
                                                      (1, 300, True, False), (5, 8, False, False)])
def test_gated_norm_of_a_recurrence_output(cuda_device, heads, dv, over_all, shared):
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(heads * dv)
    T = 6
    o = torch.randn(T, heads * dv, generator=g)
    proj = torch.randn(T, heads * dv + 7, generator=g)
    w = torch.randn(dv if shared else heads * dv, generator=g)
    for gate in ("silu", "sigmoid"):
        out = torch.empty(T, heads * dv, device=cuda_device)
        ops.gated_norm_out(o.to(cuda_device), proj.to(cuda_device), 7, w.to(cuda_device), out,
                           heads, dv, 1e-5, over_all=over_all, gate=gate, out_scale=0.7)
        od = o.double()
        if over_all:
            normed = P.rms_norm(od, w.double(), 1e-5)
        else:
            normed = P.rms_norm(od.view(T, heads, dv), w.double().view(-1, dv), 1e-5).reshape(T, -1)
        z = proj[:, 7:].double()
        want = normed * (P.silu(z) if gate == "silu" else torch.sigmoid(z)) * 0.7
        assert H.rel_err(out.cpu(), want) <= 2e-6


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("heads,kv_heads,dk,dv,conv", [
    (2, 1, 16, 32, 3), (1, 1, 40, 24, 4), (3, 3, 8, 8, 1), (2, 2, 72, 96, 2), (2, 1, 136, 20, 2),
    (1, 1, 6, 300, 5), (4, 2, 128, 64, 4), (2, 1, 320, 12, 2), (1, 1, 600, 8, 3)])
def test_delta_rule_alone(cuda_device, tmp_path, heads, kv_heads, dk, dv, conv):
    """One layer: a prompt at once, portions, and token by token, over 200 tokens, with a
    decay close to one on the first head, so that the first tokens' writes still count at
    the end."""
    raw = _one_layer(H._ket_layer("delta", H._ket_delta(heads, kv_heads, dk, dv, conv), ff=40))

    def tweak(w):
        w["l0.mix.A_log"][0] = -9.0
        w["l0.mix.dt_bias"][:] += 0.5

    d = H.make_ketopel_dir(tmp_path, "A", raw=raw, tweak=tweak, tag=f"d{heads}{dk}{dv}{conv}")
    raw, w = H.read_model_dir(d)
    reqs = {"a": H.random_tokens(200, raw["vocab"], 3), "b": H.random_tokens(37, raw["vocab"], 4)}
    ref = {r: P.forward(raw, w, t) for r, t in reqs.items()}
    for name, steps in _all_regimes(reqs, tail=150).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"delta rule {heads}x{dk}x{dv}/{name}")


@pytest.mark.parametrize("heads,dk,dv,decay", [
    (2, 16, 32, (0.9, 0.999)), (1, 40, 24, (1.0,)), (3, 8, 8, (0.5, 0.98, 0.75)),
    (2, 72, 96, (0.97, 0.99)), (1, 264, 40, (0.99,)), (1, 6, 300, (0.98,)), (1, 600, 8, (0.99,))])
def test_lightning_attention_alone(cuda_device, tmp_path, heads, dk, dv, decay):
    """One layer whose softmax branch counts for nothing."""
    layer = H._ket_parallel(H._ket_left(2, 1, 8, 8, 4), H._ket_right(heads, dk, dv, decay),
                            ls=0.0, rs=1.5)
    d = H.make_ketopel_dir(tmp_path, "A", raw=_one_layer(layer), tag=f"l{heads}{dk}{dv}")
    raw, w = H.read_model_dir(d)
    reqs = {"a": H.random_tokens(200, raw["vocab"], 3), "b": H.random_tokens(37, raw["vocab"], 4)}
    ref = {r: P.forward(raw, w, t) for r, t in reqs.items()}
    for name, steps in _all_regimes(reqs, tail=150).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"lightning {heads}x{dk}x{dv}/{name}")


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
    w["l0.norm1"][:] = 1.0
    return e_k, e_q, gen


def _stand_out_left(raw, toks, marked, amp=3.0, boost=30.0):
    """The softmax branch of a side-by-side layer: the first query head of every group
    answers ``e_q`` with a strong fixed vector in the sizes that are not rotated, and the
    group's key head answers ``e_k`` with the same vector, so that the marked query's score
    with the marked key towers over all others; the value projection is blind to both."""
    mx = raw["layers"][0]["mixer"]["left"]
    H_, G_, dk, rot = mx["heads"], mx["kv_heads"], mx["dim"], mx["rot"]["dims"]

    def tweak(w):
        p = "l0.mix.left."
        e_k, e_q, gen = _mark(w, toks, marked, amp)
        a = torch.randn(dk, generator=gen).to(w["embed"].dtype)
        a[:rot] = 0.0
        for g in range(G_):
            h0 = g * (H_ // G_)
            w[p + "q"][h0 * dk:(h0 + 1) * dk] += boost * torch.outer(a, e_q)
            w[p + "k"][g * dk:(g + 1) * dk] += boost * torch.outer(a, e_k)
        w[p + "q.norm"][:] = 1.0
        w[p + "k.norm"][:] = 1.0
        for e in (e_k, e_q):
            w[p + "v"] -= torch.outer(w[p + "v"] @ e, e)
    return tweak


def _stand_out_latent(raw, toks, marked, amp=3.0, boost=30.0):
    """Latent attention: the down projection writes ``e_k`` into the latent's first number
    (mildly: the rest of the latent still tells tokens apart), the first head's key expansion
    turns that number into a fixed vector, and the same head's query answers ``e_q`` with that
    vector, all in the sizes that are not rotated.  That head's values and the output
    projection are made large, so that what the head reads decides the logits."""
    mx = raw["layers"][0]["mixer"]
    d, dv = mx["dim"], mx["vdim"]

    def tweak(w):
        p = "l0.mix."
        e_k, e_q, gen = _mark(w, toks, marked, amp)
        a = torch.randn(d, generator=gen).to(w["embed"].dtype)
        w[p + "dkv"][0] = 0.3 * e_k
        w[p + "dkv.norm"][:] = 1.0
        w[p + "uk"][:d, 0] = a
        w[p + "q"][:d] += boost * torch.outer(a, e_q)
        w[p + "uv"][:dv] *= 6.0
        w[p + "o"] *= 4.0
    return tweak


# pages of 8: the marked key and the query that asks for it
EDGES = {"far": (3, 230), "first_token": (0, 235), "page_border": (8, 27), "page_end": (7, 24),
         "second_token": (0, 1), "neighbour": (100, 101)}


def _edge_case(cuda_device, tmp_path, raw, tweak_of, case, scale_amp=1.0):
    key, query = EDGES[case]
    toks = _distinct_tokens(240, raw["vocab"], 21)
    d = H.make_ketopel_dir(tmp_path, "A", raw=raw, tweak=tweak_of(raw, toks, (key, query)),
                           tag=case)
    raw, w = H.read_model_dir(d)
    ref = {"a": P.forward(raw, w, toks)}
    # the test is only worth something if that one key decides the query's logits: with another
    # token in the key's place they move far beyond the bound
    other = list(toks)
    other[key] = next(t for t in range(raw["vocab"]) if t not in toks)
    moved = H.rel_err(P.forward(raw, w, other)[query], ref["a"][query])
    assert moved > 100 * TOL[torch.float32], f"{case}: the key moves the logits by {moved:.3g} only"
    for name, steps in _all_regimes({"a": toks}, tail=100).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"{case}/{name}")


@pytest.mark.parametrize("case", sorted(EDGES))
def test_whole_norm_attention_alone_at_its_edges(cuda_device, tmp_path, case):
    """One layer whose lightning branch counts for nothing.  A marked key sits hundreds of
    tokens back, at the sequence's start, at a page's border or right beside its query."""
    left = H._ket_left(4, 2, 16, 24, 8, scale=0.6, softcap=25.0, scaling=(4.0, 32, 8.0, 1.0))
    raw = _one_layer(H._ket_parallel(left, H._ket_right(1, 8, 8, (0.9,)), ls=1.3, rs=0.0),
                     vocab=400)
    _edge_case(cuda_device, tmp_path, raw, _stand_out_left, case)


@pytest.mark.parametrize("case", sorted(EDGES))
def test_latent_attention_alone_at_its_edges(cuda_device, tmp_path, case):
    raw = _one_layer(H._ket_layer("latent_attention", H._ket_latent(3, 12, 8, 20, 28, scale=0.3),
                                  ff=56), vocab=400)
    _edge_case(cuda_device, tmp_path, raw, _stand_out_latent, case)


@pytest.mark.parametrize("heads,d,dr,dv,rank", [(1, 6, 2, 10, 6), (2, 40, 24, 8, 200),
                                                (5, 8, 40, 30, 12), (2, 64, 64, 128, 300)])
def test_latent_attention_sizes(cuda_device, tmp_path, heads, d, dr, dv, rank):
    """Other sizes: one head, a latent smaller than a head, a rotated part larger than the
    plain one, a latent of more than 256 numbers."""
    raw = _one_layer(H._ket_layer("latent_attention", H._ket_latent(heads, d, dr, dv, rank)),
                     width=40)
    dd = H.make_ketopel_dir(tmp_path, "B", raw=raw, tag=f"s{heads}{d}{dr}{rank}")
    raw, w = H.read_model_dir(dd)
    reqs = {"a": H.random_tokens(70, raw["vocab"], 5), "b": H.random_tokens(9, raw["vocab"], 6)}
    ref = {r: P.forward(raw, w, t) for r, t in reqs.items()}
    for name, steps in _all_regimes(reqs, tail=30).items():
        got = H.run_trace(_runner(dd, torch.float32, 4, H.peak_pages(steps, 4)), steps)
        _compare(got, ref, torch.float32, f"latent {heads}x{d}+{dr}/{rank}/{name}")


def _latent_attention_plain(q, rows, rank, scale, pos):
    """One token's heads ``q [H, W]`` over the cache rows ``rows [n, W]`` of its request, of
    which it sees ``0 .. pos``: softmax(scale q K^T) V with V the rows' first ``rank``."""
    keys = rows[:pos + 1].double()
    w = torch.softmax(q.double() @ keys.T * scale, dim=-1)
    return (w @ keys[:, :rank]).float()


@pytest.mark.parametrize("H_,rank,rot,ps", [(16, 512, 64, 16), (3, 16, 0, 8), (5, 192, 32, 64),
                                            (40, 48, 128, 16), (1, 512, 128, 32)])
def test_latent_attention_kernel_on_the_tensor_cores(cuda_device, H_, rank, rot, ps):
    """The kernel alone in bfloat16 against float arithmetic on the same rounded numbers:
    whole prompts, later portions (down to two tokens, starting inside a key tile and a page)
    and single tokens of unequal requests in one batch, over pages in a shuffled order, and a
    step of single tokens whose key tiles are shared out over CTAs (with the longest context
    given larger than it is, as a captured step has it)."""
    from binfer_b200.csrc import ops
    dev, W = cuda_device, rank + rot
    gen = torch.Generator().manual_seed(H_ * 1000 + rank)
    # (context before the step, tokens of the step)
    batches = [[(0, 70), (64, 2), (33, 130), (199, 1), (0, 1)], [(300, 1), (63, 1), (0, 1), (129, 1)],
               [(0, 257)], [(515, 1)]]
    scale = 1.7 * W ** -0.5
    for bi, reqs in enumerate(batches):
        pages_of = [(c + n + ps - 1) // ps for c, n in reqs]
        total = sum(pages_of)
        order = torch.randperm(total, generator=gen)
        cache = torch.zeros((total + 1, 1, ps, W), dtype=torch.bfloat16)
        tables = torch.full((len(reqs), max(pages_of)), -1, dtype=torch.int32)
        qs, positions, q_start, refs, at = [], [], [0], [], 0
        for b, (c, n) in enumerate(reqs):
            rows = (torch.randn((c + n, W), generator=gen) * 0.8).to(torch.bfloat16)
            mine = order[at:at + pages_of[b]]
            at += pages_of[b]
            tables[b, :pages_of[b]] = mine.to(torch.int32)
            for j in range(c + n):
                cache[mine[j // ps], 0, j % ps] = rows[j]
            q = (torch.randn((n, H_, W), generator=gen) * 1.5).to(torch.bfloat16)
            qs.append(q)
            positions += list(range(c, c + n))
            q_start.append(q_start[-1] + n)
            refs += [_latent_attention_plain(q[i].float(), rows.float(), rank, scale, c + i)
                     for i in range(n)]
        q = torch.cat(qs).to(dev)
        ref = torch.stack(refs)
        out = torch.full((q.shape[0], H_, rank), float("nan"), dtype=torch.bfloat16, device=dev)
        err = ops.error_word(dev)
        single = all(n == 1 for _, n in reqs)
        longest = max(c + n for c, n in reqs)
        for max_ctx in ([0, longest, longest + 700] if single else [0, longest]):
            out.fill_(float("nan"))
            ops.latent_attention(q, cache.to(dev), torch.tensor(q_start, dtype=torch.int32, device=dev),
                                 torch.tensor(positions, dtype=torch.int32, device=dev),
                                 tables.to(dev), out, len(reqs), max(n for _, n in reqs), H_, rank,
                                 scale, err, max_ctx=max_ctx)
            assert int(err.item()) == 0
            e = H.rel_err(out.float().cpu(), ref)
            assert e <= 1.2e-2, f"batch {bi}, longest context given as {max_ctx}: {e:.3g}"


@pytest.mark.parametrize("case", sorted(EDGES))
@pytest.mark.parametrize("which", ["whole_norm", "latent"])
def test_attention_at_its_edges_on_the_tensor_cores(cuda_device, tmp_path, which, case):
    """The marked keys again, in bfloat16 and with sizes that the tensor-core kernels take (the
    soft cap among them); the profiler shows that those kernels ran."""
    from binfer_b200.csrc import ops
    from binfer_b200.profiling import Profiler
    if which == "whole_norm":
        left = H._ket_left(4, 2, 32, 16, 16, scale=0.6, softcap=25.0, scaling=(4.0, 32, 8.0, 1.0))
        raw = _one_layer(H._ket_parallel(left, H._ket_right(1, 8, 8, (0.9,)), ls=1.3, rs=0.0),
                         vocab=400, width=64)
        from binfer_b200.parts import attention_conv_window as mod
        tweak_of, kernel = _stand_out_left, "pwm_attention"
    else:
        raw = _one_layer(H._ket_layer("latent_attention", H._ket_latent(3, 24, 16, 20, 32, scale=0.3),
                                      ff=56), vocab=400, width=64)
        from binfer_b200.parts import attention_latent as mod
        tweak_of, kernel = _stand_out_latent, "latent_attention"
    key, query = EDGES[case]
    toks = _distinct_tokens(240, raw["vocab"], 21)
    d = H.make_ketopel_dir(tmp_path, "A", torch.bfloat16, raw=raw,
                           tweak=tweak_of(raw, toks, (key, query), boost=12.0), tag=which + case)
    raw, w = H.read_model_dir(d)
    ref = {"a": P.forward(raw, w, toks)}
    other = list(toks)
    other[key] = next(t for t in range(raw["vocab"]) if t not in toks)
    moved = H.rel_err(P.forward(raw, w, other)[query], ref["a"][query])
    assert moved > 0.5, f"{case}: the key moves the logits by {moved:.3g} only"
    # a model this narrow is rounded coarsely in bfloat16 whatever the kernel: the kernel for
    # any sizes on the same rounded numbers is the sharp comparison
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
                # against the plain implementation where the marked key decides; elsewhere the
                # made-up weights (a sharp softmax, large values) magnify the rounding of the
                # cached rows alike in both kernels, and the kernels are compared below
                at_query = H.rel_err(got[name][("a", query)], ref["a"][query])
                assert at_query <= 0.25 * moved, (f"{which}/{case}/{name} (tensor cores {on}): "
                                                  f"{at_query:.3g} where the key moves {moved:.3g}")
        finally:
            ops.set_profiler(None)
            mod.TENSOR_CORES = True
        assert (kernel in seen) == on and ("paged_attention_generic" in seen) != on, sorted(seen)
        outs.append(got)
    for name in outs[0]:
        worst = max(H.rel_err(outs[0][name][k], outs[1][name][k]) for k in outs[0][name])
        assert worst <= 0.03, f"{which}/{case}/{name}: the two kernels differ by {worst:.3g}"


def test_soft_cap_and_stretched_waves_count(cuda_device, tmp_path):
    """The plain implementation first shows that leaving out the cap, the stretching or the
    larger cosines moves the logits; the engine is then held to the full form."""
    left = H._ket_left(2, 1, 16, 16, 16, scale=1.5, softcap=2.0, scaling=(16.0, 16, 4.0, 0.5))
    raw = _one_layer(H._ket_parallel(left, H._ket_right(1, 8, 8, (0.9,)), ls=1.0, rs=0.0))
    d = H.make_ketopel_dir(tmp_path, "A", raw=raw, tag="cap")
    raw, w = H.read_model_dir(d)
    toks = H.random_tokens(90, raw["vocab"], 12)
    ref = {"a": P.forward(raw, w, toks)}
    for drop in ("softcap", "scaling"):
        off = copy.deepcopy(raw)
        m = off["layers"][0]["mixer"]["left"]
        (m if drop == "softcap" else m["rot"]).pop(drop)
        assert H.rel_err(P.forward(off, w, toks), ref["a"]) > 100 * TOL[torch.float32], drop
    for name, steps in _all_regimes({"a": toks}, tail=40).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"cap and waves/{name}")


# ----------------------------------------------------------------------- whole models
LENGTHS = {"A": [5, 17, 33, 70, 121], "B": [1, 9, 40, 70, 101], "C": [3, 30, 64, 47, 2],
           "D": [2, 45, 150, 210, 90]}


def _requests(which, extra=()):
    vocab = H.KET[which]["raw"]["vocab"]
    lens = list(LENGTHS[which]) + list(extra)
    return {f"r{i}": H.random_tokens(n, vocab, 100 * i + n) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def plain_logits(tmp_path_factory):
    cache = {}

    def get(which, dtype, reqs):
        d = H.make_ketopel_dir(tmp_path_factory.getbasetemp(), which, dtype)
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
    ps = H.KET[which]["page_size"]
    runner = _runner(model_dir, dtype, ps, H.peak_pages(steps, ps))
    got = H.run_trace(runner, steps)
    assert not runner.cache.requests and all(g.pool.num_held == 0 for g in runner.cache.groups)
    assert runner.cache.slots.num_free == 4
    _compare(got, ref, dtype, f"{which}/{regime}")


def test_single_tokens_take_the_decode_kernel(cuda_device, plain_logits):
    """Steps of single tokens of the whole-norm attention (heads of 64, a soft cap, the
    branch's columns of the side-by-side buffer) run on the engine's decode kernel; with it
    switched off the tiled kernel gives the same logits up to rounding."""
    from binfer_b200.csrc import ops
    from binfer_b200.parts import attention_conv_window as mod
    from binfer_b200.profiling import Profiler
    reqs = _requests("D")
    model_dir, ref = plain_logits("D", torch.bfloat16, reqs)
    steps = H.trace_decode_tail(reqs, tail=24)
    ps = H.KET["D"]["page_size"]
    outs = []
    for on in (True, False):
        mod.DECODE_KERNEL = on
        try:
            prof = Profiler()
            got = H.run_trace(_runner(model_dir, torch.bfloat16, ps, H.peak_pages(steps, ps)), steps)
            prof.stop()
            seen = set(prof.collect())
        finally:
            ops.set_profiler(None)
            mod.DECODE_KERNEL = True
        assert ("decode_attention_persistent" in seen) == on, sorted(seen)
        assert "pwm_attention" in seen                      # the prompts' portions
        _compare(got, ref, torch.bfloat16, f"decode kernel {on}")
        outs.append(got)
    worst = max(H.rel_err(outs[0][k], outs[1][k]) for k in outs[0])
    assert worst <= 0.03, f"the two kernels differ by {worst:.3g}"


def test_long_portions_take_the_prefill_kernel(cuda_device, tmp_path):
    """Whole prompts of 300 and 280 tokens through a side-by-side layer whose softmax branch
    has heads of 128 and a soft cap run on the engine's tcgen05 prefill kernel (writing the
    scaled result into the branch's columns); with it switched off the tiled kernel gives the
    same logits up to rounding."""
    from binfer_b200.csrc import ops
    from binfer_b200.parts import attention_conv_window as mod
    from binfer_b200.profiling import Profiler
    left = H._ket_left(4, 2, 128, 128, 64, scale=0.1, softcap=4.0, scaling=(4.0, 64, 8.0, 1.0))
    raw = _one_layer(H._ket_parallel(left, H._ket_right(2, 16, 16, (0.9, 0.97)), ls=1.1, rs=0.6,
                                     ff=96), vocab=300, width=128)
    d = H.make_ketopel_dir(tmp_path, "A", torch.bfloat16, raw=raw, tag="long")
    raw, w = H.read_model_dir(d)
    reqs = {"a": H.random_tokens(300, raw["vocab"], 5), "b": H.random_tokens(280, raw["vocab"], 6)}
    ref = {rid: P.forward(raw, w, toks) for rid, toks in reqs.items()}
    steps = H.trace_whole(reqs)
    outs = []
    for on in (True, False):
        mod.DECODE_KERNEL = on
        try:
            prof = Profiler()
            got = H.run_trace(_runner(d, torch.bfloat16, 16, H.peak_pages(steps, 16)), steps)
            prof.stop()
            seen = set(prof.collect())
        finally:
            ops.set_profiler(None)
            mod.DECODE_KERNEL = True
        assert ("prefill_attention_umma2" in seen) == on and ("pwm_attention" in seen) != on, sorted(seen)
        _compare(got, ref, torch.bfloat16, f"prefill kernel {on}")
        outs.append(got)
    worst = max(H.rel_err(outs[0][k], outs[1][k]) for k in outs[0])
    assert worst <= 0.03, f"the two kernels differ by {worst:.3g}"


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_the_stream_after_every_layer_run(cuda_device, plain_logits, which):
    """The residual stream after each run of a layer, the looped ones each time: what a pass
    starts with is added once, right before its first layer."""
    from binfer_b200.engine.runner import StepItem
    toks = H.random_tokens(19, H.KET[which]["raw"]["vocab"], 77)
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
        assert H.rel_err(g.cpu(), r) <= 2e-5, f"{which}: after layer run {i}"


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_regimes_agree_bitwise_in_float32(cuda_device, plain_logits, which):
    """Every sum's order depends on positions alone: cutting and batching change no bit."""
    reqs = _requests(which)
    model_dir, _ = plain_logits(which, torch.float32, reqs)
    ps = H.KET[which]["page_size"]
    outs = []
    for steps in _all_regimes(reqs).values():
        outs.append(H.run_trace(_runner(model_dir, torch.float32, ps, H.peak_pages(steps, ps)),
                                steps))
    for other in outs[1:]:
        for key, row in outs[0].items():
            assert torch.equal(row, other[key]), f"{which}: logits at {key} depend on the cut"


def test_long_decoding(cuda_device, plain_logits):
    """A short prompt, then 300 tokens one by one."""
    which, dtype = "B", torch.float32
    reqs = {"long": H.random_tokens(304, H.KET[which]["raw"]["vocab"], 7)}
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
    ps = H.KET[which]["page_size"]
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
    d = H.make_ketopel_dir(tmp_path, "A")
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


def test_command_line_generates_from_a_looped_folder(cuda_device, tmp_path, capsys):
    """``bin/binfer``'s entry point on a looped folder: the registry picks the family from
    config.json; greedy tokens are the plain implementation's, and sampling with a seed
    gives the same tokens twice."""
    from binfer_b200.cli import main
    d = H.make_ketopel_dir(tmp_path, "C")
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
    """``bin/trace_run`` as a user runs it on a looped model: six requests through its four
    state slots and a page pool sized by ``--max-tokens``."""
    import test_trace_run_gpu as TR
    d = H.make_ketopel_dir(tmp_path, "B")
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
