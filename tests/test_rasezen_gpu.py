"""Rasezen in the engine against the plain implementation (tests/plain_rasezen.py): every
mechanism alone, then whole prompts, prompts in portions, decoding token by token, batches of
unequal requests, slots, pages and state that are used again, and greedy generation through the
library's entry point."""
import json

import pytest
import torch

import plain_rasezen as P
from rasezen_models import SMALL, attention, config, dense, layer, make_weights, moe, state_space, write_model

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
DTYPES = ["float32", "bfloat16"]


def tol(dtype):
    return 3e-5 if dtype in (F32, "float32") else 3e-2


def close(got, ref, dtype, what="", stray_rows=0.0):
    """Largest difference against the reference's scale. `stray_rows`: the share of rows that may
    be further off (a bfloat16 run can choose another expert for a token whose two best scores
    lie within rounding of each other); no row may be wildly off."""
    got, ref = got.detach().float().cpu(), ref.float()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what
    scale = max(1.0, float(ref.abs().max()))
    err = (got - ref).abs().reshape(got.shape[0], -1).max(dim=1).values / scale
    if stray_rows and dtype not in (F32, "float32"):
        over = int((err > tol(dtype)).sum())
        assert over <= max(1, int(stray_rows * err.numel())) and float(err.max()) < 0.5, \
            f"{what}: {over} of {err.numel()} rows over {tol(dtype):.1e}, worst {float(err.max()):.3e}"
        return
    assert float(err.max()) <= tol(dtype), f"{what}: {float(err.max()):.3e} > {tol(dtype):.1e} (row {int(err.argmax())})"


def runtime(dtype):
    from lumenllm_b200.parts import Runtime
    return Runtime(torch.device("cuda", 0), {"float32": F32, "bfloat16": BF16}.get(dtype, dtype))


def tokens_of(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: write_model(cfg, tmp_path_factory.mktemp(f"rasezen{name}"), seed=60 + i)
            for i, (name, cfg) in enumerate(SMALL.items())}


@pytest.fixture(scope="module")
def plain(models):
    """name -> (config, float32 weights, cache of plain logits by token tuple)."""
    return {name: (*P.load_model(folder), {}) for name, folder in models.items()}


def plain_logits(plain, name, tokens):
    cfg, w, memo = plain[name]
    key = tuple(tokens)
    if key not in memo:
        memo[key] = P.forward(cfg, w, list(tokens))
    return memo[key]


def engine_of(models, name, dtype, **kw):
    from lumenllm_b200.engine import Engine
    kw.setdefault("max_tokens", 4096)
    return Engine.from_folder(models[name], dtype=dtype, **kw)


def part_of(category, kind, params, prefix, weights, dtype):
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.parts import build_part
    return build_part(category, PartSpec(kind, params, prefix=prefix), {k: v.cuda() for k, v in weights.items()},
                      runtime(dtype))


def one_layer(mixer, mlp, D, seed, edit=None):
    """(config, bfloat16 weights, the same as float32 on the CPU) of a one-layer model."""
    cfg = config(8, D, 1e-6, [layer(mixer, mlp)])
    w = make_weights(cfg, seed)
    if edit is not None:
        edit(w)
    return cfg, w, {k: v.float() for k, v in w.items()}


def run_mixer(mixer, rt, pieces_by_seq, order=None):
    """Feeds sequences' rows piece by piece through a mixer alone. pieces_by_seq: for each sequence
    a list of row blocks (an empty block: the sequence pauses that step). Returns each sequence's
    updates in order."""
    from lumenllm_b200.cache import KVCache
    from lumenllm_b200.engine.context import EntryView, StepEntry, build_context
    need, shape = mixer.cache_need(), mixer.state_shape()
    cache = KVCache({0: need} if need is not None else {}, 4096, 4, 4096, dtype=rt.dtype, device=rt.device,
                    state_shapes={0: shape} if shape is not None else None)
    outs = [[] for _ in pieces_by_seq]
    for round_ in range(2 if order == "twice" else 1):       # the second round takes the first round's slots
        slots = [cache.alloc_slot() for _ in pieces_by_seq]
        outs = [[] for _ in pieces_by_seq]
        for step in range(max(len(p) for p in pieces_by_seq)):
            live = [b for b, p in enumerate(pieces_by_seq) if step < len(p) and p[step].shape[0]]
            if not live:
                continue
            ctx, _ = build_context(cache, rt, [StepEntry(slots[b], [0] * pieces_by_seq[b][step].shape[0]) for b in live])
            y = torch.cat([pieces_by_seq[b][step] for b in live]).to(rt.dtype).cuda()
            out = mixer.forward(y, ctx, EntryView(ctx, 0, 0 if need is not None else None, True))
            out = (out.sum(0) if out.dim() == 3 else out).cpu()
            at = 0
            for b in live:
                n = pieces_by_seq[b][step].shape[0]
                outs[b].append(out[at:at + n])
                cache.commit(slots[b], n)
                at += n
        for s in slots:
            cache.free_slot(s)
        cache.check()
    return [torch.cat(o) for o in outs]


def cut(y, sizes):
    out, at = [], 0
    for n in sizes:
        out.append(y[at:at + n])
        at += n
    assert at == y.shape[0]
    return out


# ------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("dtype", [F32, BF16])
def test_norm_with_one_number_as_weight(dtype):
    from lumenllm_b200.engine.model import expected_tensors  # noqa: F401  (registers the parts)
    D = 72
    g = torch.Generator().manual_seed(1)
    w = {"n": torch.tensor(1.37).to(BF16)}
    norm = part_of("norm", "rmsnorm", {"size": D, "eps": 1e-5, "tensor": "n", "scalar": True}, "", w, dtype)
    h, delta = torch.randn(9, D, generator=g) * 3, torch.randn(4, 9, D, generator=g)
    ref = P.scalar_norm(h + delta.sum(0), w["n"].float(), 1e-5)
    hd = h.cuda()
    got = norm.forward(hd, delta.cuda(), dtype)
    close(got, ref, dtype)
    close(hd, h + delta.sum(0), F32)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_xielu(dtype):
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(2)
    z = torch.randn(3, 11, 50, generator=g) * 2
    z[0, 0, :6] = torch.tensor([0.0, -30.0, 30.0, -1e-4, 1e-4, -0.5]) - z[1:, 0, :6].sum(0)
    for p, q in ((0.3, -0.2), (-4.0, 5.0), (0.0, 0.0)):
        act = torch.tensor([p, q])
        ref = P.xielu(z.sum(0), act[0], act[1])
        close(K.xielu(z.cuda(), act.cuda(), dtype), ref, dtype, f"p {p} q {q}")


ATTENTIONS = [attention(4, 2, 16, 24, 0.3, size=9, rot=8), attention(6, 6, 32, 32, 0.11, rot=32, base=1e6),
              attention(3, 1, 32, 16, 0.2, size=1000), attention(2, 2, 64, 64, 0.15, size=33, rot=64),
              attention(5, 5, 24, 8, 0.5, size=1, rot=2), attention(2, 1, 128, 128, 0.1, size=70, rot=32),
              attention(3, 3, 40, 72, 0.2, size=64, rot=40, base=77.0), attention(34, 1, 20, 10, 0.4, size=50, rot=4),
              attention(2, 1, 64, 128, 0.12, size=90, rot=16), attention(40, 2, 64, 64, 0.12, size=100, rot=64)]


def attention_part(m, D, dtype, seed, edit=None):
    from lumenllm_b200.config import PartSpec
    _, w, wf = one_layer(m, None, D, seed, edit)
    rot = m.get("rot")
    position = PartSpec("rotary", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": rot["base"],
                                   "wide_frequencies": True}) if rot else PartSpec("none", {})
    params = {"hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
              "value_dim": m["vdim"], "softmax_scale": m["scale"], "window": m["mask"]["size"] if "mask" in m else 0,
              "norm_eps": 1e-6, "value_norm": True, "position": position}
    return part_of("mixer", "wide_norm_attention", params, "l0.mix", w, dtype), wf


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", ATTENTIONS)
def test_attention_part(m, dtype):
    """The mixer alone: a prompt, then the same sequence continued in portions and token by token."""
    D, T = 48, 150
    mixer, w = attention_part(m, D, dtype, seed=5)
    y = torch.randn(T, D, generator=torch.Generator().manual_seed(6)).to(dtype).float()
    ref = P.attention(y, w, "l0.mix", m, 1e-6)
    got = run_mixer(mixer, runtime(dtype), [cut(y, [100, 2, 29] + [1] * 19)])[0]
    close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_attention_of_several_sequences_at_once(dtype):
    m = attention(4, 2, 32, 16, 0.2, size=40, rot=16)
    D = 40
    mixer, w = attention_part(m, D, dtype, seed=9)
    g = torch.Generator().manual_seed(10)
    ys = [torch.randn(n, D, generator=g).to(dtype).float() for n in (90, 5, 131)]
    refs = [P.attention(y, w, "l0.mix", m, 1e-6) for y in ys]
    pieces = [cut(ys[0], [70, 1, 19]), cut(ys[1], [1, 0, 4]), cut(ys[2], [0, 128, 3])]
    for got, ref in zip(run_mixer(mixer, runtime(dtype), pieces, order="twice"), refs):
        close(got, ref, dtype)


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_loud_key_at_every_edge_of_sight(dtype, decode):
    """Queries are the (normed) inputs themselves and keys the inputs shifted by seven channels,
    and one earlier token is made loud so that its KEY points where the last QUERY points: this
    single key takes nearly all of the query's weight where it is in sight and none where it is
    not: far back among hundreds of keys, on both sides of the window's edge, on both sides of
    page borders, and at the sequence's first token. Beside the window's edge stands the mask that
    differs by one: the plain result under it must be far from the right one, else the case would
    show nothing."""
    H, d, D, T, size = 2, 32, 64, 300, 130

    def identity(w):
        for name in ("q", "k", "v"):
            w["l0.mix." + name] = torch.eye(D).to(BF16)
            w["l0.mix." + name + ".b"] = torch.zeros(D).to(BF16)
        w["l0.mix.k"] = torch.roll(torch.eye(D), 7, dims=0).to(BF16)
        w["l0.mix.q.norm"] = w["l0.mix.k.norm"] = torch.ones(D).to(BF16)
    g = torch.Generator().manual_seed(8)
    u = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
    query = T - 1
    lo = query - size + 1
    for window, loud, wrong_window in [(size, lo - 1, size + 1), (size, lo, size - 1), (size, 191, None), (size, 192, None),
                                       (size, 255, None), (size, 256, None), (size, query - 1, None), (None, 0, None),
                                       (None, 63, None), (None, 64, None), (T, 0, T - 1), (T - 1, 0, T)]:
        m = attention(H, H, d, d, 1.0, size=window)
        mixer, w = attention_part(m, D, dtype, seed=7, edit=identity)
        y = torch.randn(T, D, generator=g) * 0.3
        y[loud] += 12 * torch.roll(u, -7)
        y[query] += 12 * u
        y = y.to(dtype).float()
        ref = P.attention(y, w, "l0.mix", m, 1e-6)
        if wrong_window is not None:
            wrong = P.attention(y, w, "l0.mix", attention(H, H, d, d, 1.0, size=wrong_window), 1e-6)
            assert float((wrong[query] - ref[query]).abs().max()) > 10 * tol(BF16) * max(1.0, float(ref.abs().max()))
        pieces = cut(y, [T - 40] + [1] * 40) if decode else [y]
        close(run_mixer(mixer, runtime(dtype), [pieces])[0], ref, dtype, f"window {window}, loud key {loud}")


SPACES = [state_space(4, 16, 8, 1, 4, 1), state_space(6, 8, 40, 3, 2, 3), state_space(2, 24, 16, 2, 1, 4),
          state_space(4, 32, 100, 2, 3, 2), state_space(1, 7, 5, 1, 16, 1), state_space(3, 64, 128, 3, 5, 6)]


def state_space_part(m, D, dtype, seed, edit=None):
    _, w, wf = one_layer(m, None, D, seed, edit)
    params = {"hidden_size": D, "num_heads": m["heads"], "head_dim": m["vdim"], "state_size": m["state"],
              "groups": m["groups"], "taps": m["conv"], "norm_groups": m["norm_groups"], "norm_eps": 1e-6}
    return part_of("mixer", "mamba2", params, "l0.mix", w, dtype), wf


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", SPACES)
def test_state_space_part_in_any_portions(m, dtype):
    """Two sequences fed in unequal portions (down to one token, one of them pausing) give what
    the whole sequences give, convolution state and recurrent state carried across every cut; the
    slots' next users start from zeros."""
    D = 40
    mixer, w = state_space_part(m, D, dtype, seed=11)
    g = torch.Generator().manual_seed(12)
    ys = [torch.randn(n, D, generator=g).to(dtype).float() for n in (61, 23)]
    refs = [P.state_space(y, w, "l0.mix", m, 1e-6) for y in ys]
    pieces = [cut(ys[0], [1, 1, 2, 37, 0, 20]), cut(ys[1], [3, 0, 1, 1, 17, 1])]
    for got, ref in zip(run_mixer(mixer, runtime(dtype), pieces, order="twice"), refs):
        close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_the_recurrence_remembers_far_back(dtype):
    """With a decay close to one and a loud early token, what the state holds of that token
    decides the outputs hundreds of tokens later: whole, in portions and decoded one by one. A
    state that was lost or restarted on the way shows (the plain result without the early token
    is far from the right one)."""
    m = state_space(2, 16, 24, 1, 2, 1)
    D, T = 32, 420

    def slow(w):
        w["l0.mix.A_log"] = torch.full((2,), -7.0).to(BF16)
        w["l0.mix.dt_bias"] = torch.full((2,), -1.0).to(BF16)
    mixer, w = state_space_part(m, D, dtype, seed=13, edit=slow)
    g = torch.Generator().manual_seed(14)
    y = torch.randn(T, D, generator=g) * 0.2
    y[3] *= 40
    y = y.to(dtype).float()
    ref = P.state_space(y, w, "l0.mix", m, 1e-6)
    quiet = y.clone()
    quiet[3] /= 40
    assert float((P.state_space(quiet, w, "l0.mix", m, 1e-6)[-1] - ref[-1]).abs().max()) > 0.3 * float(ref[-1].abs().max())
    for sizes in ([T], [200, 2, 2, 150, 66], [380] + [1] * 40):
        close(run_mixer(mixer, runtime(dtype), [cut(y, sizes)])[0], ref, dtype, f"cut as {sizes[:4]}")


def test_router_choices_and_weights():
    """The correction moves the choice and not the weight; identity experts are indices like
    any other; equal scores go to the lower index; weights are not renormalised."""
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(15)
    for E, top in ((5, 2), (10, 3), (3, 3), (70, 8), (1, 1)):
        logits = torch.randn(33, E, generator=g) * 2
        corr = torch.randn(E, generator=g) * 0.3
        logits[0] = 0.0                                  # all equal: the correction alone decides
        w = {"r.router": torch.eye(E), "r.correction": corr}
        idx_ref, wt_ref = P.route(logits, w, "r", {"top": top, "scale": 1.75})
        idx, wt = K.moe_route(logits.cuda(), corr.cuda(), top, 1.75)
        assert torch.equal(idx.cpu().long(), idx_ref), (E, top)
        assert float((wt.cpu() - wt_ref).abs().max()) < 1e-6
    logits = torch.tensor([[1.0, 3.0, 3.0, 0.0]])
    idx, wt = K.moe_route(logits.cuda(), None, 2, 1.0)
    assert idx.cpu().tolist() == [[1, 2]]
    idx, wt = K.moe_route(logits.cuda(), torch.tensor([5.0, 0.0, 0.0, 0.0]).cuda(), 1, 2.0)
    s = torch.softmax(logits, -1)
    assert idx.cpu().tolist() == [[0]] and abs(float(wt[0, 0]) - 2.0 * float(s[0, 0])) < 1e-6


MIXTURES = [moe(24, 4, 1, 2, 1.5, shared=32), moe(40, 3, 0, 1, 1.0), moe(16, 5, 2, 3, 0.7, shared=8),
            moe(8, 40, 0, 4, 2.0), moe(72, 2, 3, 5, 1.0, shared=100), moe(20, 3, 1, 2, 1.0, shared=12)]


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("mlp", MIXTURES)
def test_routed_experts_part(mlp, dtype):
    """One token, a few, and more tokens than a row tile an expert; experts that nobody chose."""
    D = 56
    cfg, w, wf = one_layer(attention(1, 1, 8, 8, 1.0), mlp, D, seed=16)
    r = mlp["router"]
    part = part_of("ffn", "routed_experts", {
        "hidden_size": D, "expert_size": mlp["expert"]["ff"], "num_experts": r["experts"],
        "identity_experts": r["identity"], "top": r["top"], "scale": r["scale"],
        "shared_size": mlp["shared"]["ff"] if "shared" in mlp else 0}, "l0.mlp", w, dtype)
    g = torch.Generator().manual_seed(17)
    for n in (1, 7, 300):
        y = torch.randn(n, D, generator=g).to(dtype).float()
        ref = P.expert_mixture(y, wf, "l0.mlp", mlp)
        out = part.forward(y.to(dtype).cuda(), None)
        assert out.shape[0] >= r["top"]
        close(out.sum(0), ref, dtype, f"{n} tokens", stray_rows=0.02)


# ------------------------------------------------------------------ the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_whole_prompts(name, dtype, models, plain):
    from lumenllm_b200.engine import StepEntry
    eng = engine_of(models, name, dtype)
    for toks in tokens_of(SMALL[name], (1, 2, 37, 201) + ((640,) if name == "Z" else ()), seed=1):
        slot = eng.alloc_slot()
        got = eng.step([StepEntry(slot, toks, list(range(len(toks))))])
        eng.free_slot(slot)
        close(got, plain_logits(plain, name, toks), dtype, f"{name} {len(toks)} tokens", stray_rows=0.03)
    eng.check_kernels()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_model_whose_rows_are_no_multiples_of_16_bytes(dtype, tmp_path):
    """Width 44, heads of 6 keys and 10 values, 7 channels a state-space head, experts of 9: no row
    of any matrix is a multiple of 16 bytes, so the products go the ways that need no alignment."""
    from lumenllm_b200.engine import Engine, StepEntry
    cfg = config(61, 44, 1e-5, [layer(attention(3, 1, 6, 10, 0.4, size=20, rot=4), moe(9, 3, 1, 2, 1.2, shared=5)),
                                layer(state_space(2, 7, 9, 1, 3, 2), dense(30))])
    folder = write_model(cfg, tmp_path / "m", seed=90)
    _, w = P.load_model(folder)
    toks = tokens_of(cfg, (90,), seed=91)[0]
    ref = P.forward(cfg, w, toks)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=2)
    slot = eng.alloc_slot()
    got = [eng.step([StepEntry(slot, toks[:70], list(range(70)))])]
    got += [eng.step([StepEntry(slot, [toks[t]], [0])]) for t in range(70, 90)]
    close(torch.cat(got), ref, dtype, stray_rows=0.03)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_model_without_attention(dtype, tmp_path):
    """Only state-space layers: no cache group at all, the sequences' state is everything that is
    kept; a prompt, portions, single tokens, and two requests in a batch."""
    from lumenllm_b200.engine import Engine, StepEntry
    cfg = config(50, 48, 1e-5, [layer(state_space(3, 16, 12, 3, 2, 1), dense(40)),
                                layer(state_space(2, 8, 36, 1, 3, 2), None)])
    folder = write_model(cfg, tmp_path / "m", seed=80)
    _, w = P.load_model(folder)
    a, b = tokens_of(cfg, (150, 40), seed=81)
    ra, rb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=2)
    assert not eng.cache.groups
    sa, sb = eng.alloc_slot(), eng.alloc_slot()
    got = eng.step([StepEntry(sa, a[:100], list(range(100))), StepEntry(sb, b[:7], list(range(7)))])
    close(got, torch.cat([ra[:100], rb[:7]]), dtype)
    got = eng.step([StepEntry(sa, a[100:103], [0, 1, 2]), StepEntry(sb, b[7:39], list(range(32)))])
    close(got, torch.cat([ra[100:103], rb[7:39]]), dtype)
    rows = [eng.step([StepEntry(sa, [a[t]], [0])] + ([StepEntry(sb, [b[39]], [0])] if t == 103 else []))
            for t in range(103, 150)]
    close(torch.cat([r[:1] for r in rows]), ra[103:], dtype)
    close(rows[0][1:], rb[39:], dtype)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_residual_stream_after_every_layer(name, dtype, models, plain):
    """Layer by layer: the stream with each layer's two updates added, against the plain one."""
    from lumenllm_b200.engine import StepEntry
    from lumenllm_b200.engine.context import EntryView
    cfg, w, _ = plain[name]
    toks = tokens_of(cfg, (45,), seed=2)[0]
    _, streams = P.forward(cfg, w, toks, return_layers=True)
    eng = engine_of(models, name, dtype)
    slot = eng.alloc_slot()
    ctx = eng.build_context([StepEntry(slot, toks)])
    h, pending = eng.model.embedding.forward(ctx.tokens, ctx), None
    for i, e in enumerate(eng.model.schedule):
        view = EntryView(ctx, i, i if i in ctx.cache.group_of else None, True)
        h, pending = eng.model.blocks[e.layer].forward(h, pending, ctx, view)
        x = h if pending is None else h + (pending.sum(0) if pending.dim() == 3 else pending)
        close(x, streams[i], dtype, f"{name} after layer {i}", stray_rows=0.05)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_prompt_in_portions_and_decoded_token_by_token(name, dtype, models, plain):
    from lumenllm_b200.engine import StepEntry
    toks = tokens_of(SMALL[name], (230,), seed=3)[0]
    ref = plain_logits(plain, name, toks)
    eng = engine_of(models, name, dtype)
    for cuts in ([2, 2, 3, 60, 1, 64, 5, 93], [127, 1, 1, 101], [100] + [1] * 130):
        slot = eng.alloc_slot()
        got, at = [], 0
        for n in cuts:
            got.append(eng.step([StepEntry(slot, toks[at:at + n], list(range(n)))]))
            at += n
        eng.free_slot(slot)
        close(torch.cat(got), ref[:at], dtype, f"{name} cut as {cuts[:4]}...", stray_rows=0.03)
    eng.check_kernels()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_a_batch_of_unequal_requests_equals_each_alone(name, dtype, models, plain):
    """Prompts of unequal lengths in one step, then decoded together while the shorter requests
    leave; their slots, pages and state rows go to a second batch at once."""
    from lumenllm_b200.engine import StepEntry
    eng = engine_of(models, name, dtype, max_tokens=1024, max_slots=4)
    lens, tail = (1, 66, 140, 17), (3, 30, 12, 20)
    for round_ in range(2):
        seqs = tokens_of(SMALL[name], [n + t for n, t in zip(lens, tail)], seed=10 + round_)
        refs = [plain_logits(plain, name, s) for s in seqs]
        slots = [eng.alloc_slot() for _ in seqs]
        got = eng.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lens)])
        close(got, torch.cat([r[:n] for r, n in zip(refs, lens)]), dtype, f"{name} prompts", stray_rows=0.03)
        live = list(range(len(seqs)))
        rows, want = [], []
        for t in range(max(tail)):
            live = [b for b in live if t < tail[b]]
            rows.append(eng.step([StepEntry(slots[b], [seqs[b][lens[b] + t]], [0]) for b in live]))
            want.append(torch.stack([refs[b][lens[b] + t] for b in live]))
            for b in [b for b in live if t + 1 == tail[b]]:
                eng.free_slot(slots[b])
        close(torch.cat(rows), torch.cat(want), dtype, f"{name} decoded together", stray_rows=0.03)
        eng.cache.check()
        assert not eng.cache.slots.held
    eng.check_kernels()


@pytest.mark.parametrize("name", ["X", "Z"])
def test_decoded_logits_do_not_depend_on_the_batch(name, models):
    """The same request decoded alone and among others: the same bits, in both precisions."""
    from lumenllm_b200.engine import StepEntry
    for dtype in DTYPES:
        eng = engine_of(models, name, dtype)
        seqs = tokens_of(SMALL[name], (90, 150, 31), seed=20)

        def run(members):
            slots = {b: eng.alloc_slot() for b in members}
            eng.step([StepEntry(slots[b], seqs[b][:-8]) for b in members])
            rows = []
            for t in range(8):
                out = eng.step([StepEntry(slots[b], [seqs[b][len(seqs[b]) - 8 + t]], [0]) for b in members])
                rows.append(out[members.index(0)].clone())
            for s in slots.values():
                eng.free_slot(s)
            return torch.stack(rows)
        assert torch.equal(run([0]), run([1, 0, 2])), (name, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_while_windows_pass_and_pages_go(dtype, models, plain):
    """A request decoded one token at a time over several pages: the windows (9 and 70 keys) pass
    over decoded tokens and page borders, windowed layers hold few pages at a time, and the
    recurrent layers carry their state all the way."""
    from lumenllm_b200.cache import PAGE
    from lumenllm_b200.engine import StepEntry
    name = "X"
    toks = tokens_of(SMALL[name], (3 * PAGE + 20,), seed=30)[0]
    ref = plain_logits(plain, name, toks)
    eng = engine_of(models, name, dtype, max_tokens=6 * PAGE, max_slots=2)
    slot = eng.alloc_slot()
    got = [eng.step([StepEntry(slot, toks[:5], list(range(5)))])]
    for t in range(5, len(toks)):
        got.append(eng.step([StepEntry(slot, [toks[t]], [0])]))
        assert all(g.n_held[slot] <= 3 for g in eng.cache.groups)
    close(torch.cat(got), ref, dtype, stray_rows=0.03)
    other = eng.alloc_slot()                      # the pages given back serve another request meanwhile
    got = eng.step([StepEntry(other, toks[:2 * PAGE], [2 * PAGE - 1])])
    close(got, ref[2 * PAGE - 1:2 * PAGE], dtype, stray_rows=0.03)
    eng.free_slot(slot)
    eng.free_slot(other)
    eng.cache.check()
    eng.check_kernels()


def test_a_long_prompt_whose_products_add_into_the_stream(tmp_path):
    """A prompt long and wide enough for the output products to add their result to the residual
    stream in their epilogue (no update is handed on then), both sublayers of a block still
    reading the same normed rows."""
    from lumenllm_b200.engine import Engine, StepEntry
    from lumenllm_b200.ops import kernels as K
    cfg = config(64, 1024, 1e-6, [
        layer(attention(4, 2, 64, 64, 0.125, size=300, rot=64), dense(512)),
        layer(state_space(16, 64, 16, 2, 3, 4), moe(128, 4, 1, 2, 1.5, shared=256))])
    T = 4900
    assert K.gemm_tc_adds(T, 1024)
    folder = write_model(cfg, tmp_path / "wide", seed=70)
    toks = tokens_of(cfg, (T,), seed=71)[0]
    want = [0, 1, 299, 300, 301, 2047, T - 2, T - 1]
    _, w = P.load_model(folder)
    ref = P.forward(cfg, w, toks)[want]
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=8192)
    slot = eng.alloc_slot()
    got = eng.step([StepEntry(slot, toks, want)])
    close(got, ref, "bfloat16", stray_rows=0.13)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, models, plain):
    """build(EngineConfig).generate: batches, the scheduler's run-ahead and captured steps."""
    from lumenllm_b200 import EngineConfig, GenerateRequest, build
    name = "Z"
    cfg, w, _ = plain[name]
    built = build(EngineConfig(model_path=str(models[name]), dtype=dtype, context_size=512, max_batch=3))
    assert built.engine.model.graph_safe
    prompts = tokens_of(cfg, (70, 3, 29, 130), seed=40)
    outs = built.generate([GenerateRequest(p, 10) for p in prompts], eos_token_ids=[])
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and len(o.tokens) == 10
        lg = P.forward(cfg, w, list(p) + o.tokens)
        for k, tok in enumerate(o.tokens):
            row = lg[len(p) - 1 + k]
            gap = float(row.max() - row[tok])     # 0 where the plain choice was made
            assert gap <= (1e-4 if dtype == "float32" else 0.05 * max(1.0, float(row.abs().max()))), (k, gap)
        if dtype == "float32":
            assert o.tokens == P.generate_greedy(cfg, w, p, 10)
    built.engine.check_kernels()


def test_command_line_generates(models, capsys):
    from lumenllm_b200.cli import main
    rc = main(["generate", "--model", str(models["X"]), "--prompt-tokens", "5,6,7", "--prompt-tokens", "1",
               "--max-tokens", "4", "--ctx-size", "128", "--format", "json", "--dtype", "float32"])
    assert rc == 0
    outs = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    cfg, w = P.load_model(models["X"])
    assert [o["tokens"] for o in outs] == [P.generate_greedy(cfg, w, p, 4) for p in ([5, 6, 7], [1])]


def test_trace_replay(models, plain, tmp_path):
    """bin/trace_run on a model of this design: prompts in one batch, decoded together, portions."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    name = "Y"
    toks = tokens_of(SMALL[name], (40, 75), seed=50)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[0][:30], "want": [0, 29]},
                                     {"id": "b", "tokens": toks[1][:70], "want": [69]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[0][30:31], "want": [0]},
                                     {"id": "b", "tokens": toks[1][70:71], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[0][31:40], "want": [8]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": toks[1][71:75], "want": [0, 3]}], "end": ["b"]}]
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(models[name]), "--dtype",
                        "float32", "--out", str(out), "--max-tokens", "256"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain_logits(plain, name, toks[0]), plain_logits(plain, name, toks[1])
    V = SMALL[name]["vocab"]
    read = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4")).view(-1, V)
    close(read(0), torch.stack([ra[0], ra[29], rb[69]]), "float32")
    close(read(1), ra[30:31], "float32")
    close(read(2), ra[39:40], "float32")
    close(read(3), torch.stack([rb[71], rb[74]]), "float32")
