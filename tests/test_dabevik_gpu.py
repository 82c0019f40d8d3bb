"""Dabevik in the engine against the plain implementation (tests/plain_dabevik.py): every
mechanism alone, then whole prompts, prompts in portions, decoding token by token, batches of
unequal requests, slots and pages that are used again, and greedy generation through the
library's entry point."""
import json

import pytest
import torch

import plain_dabevik as P
from dabevik_models import SMALL, attention, config, layer, make_weights, write_model

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
DTYPES = ["float32", "bfloat16"]


def tol(dtype):
    return 3e-5 if dtype in (F32, "float32") else 3e-2


def close(got, ref, dtype, what=""):
    got, ref = got.detach().float().cpu(), ref.float()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what
    err, scale = float((got - ref).abs().max()), max(1.0, float(ref.abs().max()))
    assert err <= tol(dtype) * scale, f"{what}: {err:.3e} > {tol(dtype) * scale:.3e}"


def runtime(dtype):
    from lumenllm_b200.parts import Runtime
    return Runtime(torch.device("cuda", 0), dtype)


def tokens_of(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(SMALL.items()):
        out[name] = write_model(cfg, tmp_path_factory.mktemp(f"dabevik{name}"), seed=40 + i)
    return out


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


# ------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("tiled", [False, True])
def test_embedding_scaled_with_learned_positions(tiled):
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(0)
    table = torch.randn(50, 72, generator=g).to(BF16)
    pos = torch.randn(30, 72, generator=g).to(BF16)
    tok = torch.tensor([0, 49, 7, 7, 13], dtype=torch.int32)
    at = torch.tensor([0, 29, 1, 2, 17], dtype=torch.int32)
    ref = P.embed(tok.long(), table.float(), 5.25, pos.float(), at.long())
    t = K.tile_weight(table.cuda()) if tiled else table.cuda()
    got = K.embed_pos(tok.cuda(), t, 5.25, at.cuda(), pos.cuda())
    assert torch.equal(got.cpu(), ref)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_input_convolution_in_any_portions(taps):
    """Two sequences fed in unequal portions (down to one token, one sequence pausing) give what
    the whole sequences give; a slot that is handed out again starts from zeros."""
    from lumenllm_b200.cache import KVCache
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.engine.context import StepEntry, build_context
    from lumenllm_b200.parts import build_part
    rt = runtime(F32)
    D = 40
    g = torch.Generator().manual_seed(taps)
    w = {"c": torch.randn(D, taps, generator=g).to(BF16).cuda()}
    part = build_part("input_conv", PartSpec("causal_depthwise", {"size": D, "taps": taps, "tensor": "c"}), w, rt)
    shapes = {(0, "block"): ((taps - 1, D), F32)} if taps > 1 else {}
    cache = KVCache({}, 4096, 4, 4096, dtype=F32, device=rt.device, state_shapes=shapes)
    for round_ in range(2):
        seqs = [torch.randn(n, D, generator=g) for n in (23, 9)]
        refs = [P.input_convolution(s, w["c"].float().cpu()) for s in seqs]
        slots = [cache.alloc_slot(), cache.alloc_slot()]
        cuts = [[1, 1, 2, 7, 0, 12], [3, 0, 1, 1, 4, 0]]
        at = [0, 0]
        for step in range(6):
            entries, want = [], []
            for b in range(2):
                n = cuts[b][step]
                if n:
                    entries.append(StepEntry(slots[b], [0] * n))
                    want.append((b, at[b], n))
            ctx, _ = build_context(cache, rt, entries)
            y = torch.cat([seqs[b][a:a + n] for b, a, n in want]).cuda()
            out = part.forward(y, cache.state.of(0, "block"), ctx, F32).cpu()
            ref = torch.cat([refs[b][a:a + n] for b, a, n in want])
            assert float((out - ref).abs().max()) < 1e-5, (taps, round_, step)
            for e, (b, a, n) in zip(entries, want):
                cache.commit(e.slot, n)
                at[b] += n
        for s in slots:
            cache.free_slot(s)


@pytest.mark.parametrize("taps", [1, 3, 8, 11])
def test_input_convolution_of_long_prompts(taps):
    """Steps of many tokens (blocks then take several tokens each, up to eight taps): sequences
    that start and continue inside the step, their borders anywhere among the blocks' tokens."""
    from lumenllm_b200.cache import KVCache
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.engine.context import StepEntry, build_context
    from lumenllm_b200.parts import build_part
    rt = runtime(F32)
    D = 72
    g = torch.Generator().manual_seed(100 + taps)
    w = {"c": torch.randn(D, taps, generator=g).to(BF16).cuda()}
    part = build_part("input_conv", PartSpec("causal_depthwise", {"size": D, "taps": taps, "tensor": "c"}), w, rt)
    shapes = {(0, "block"): ((taps - 1, D), F32)} if taps > 1 else {}
    cache = KVCache({}, 8192, 4, 8192, dtype=F32, device=rt.device, state_shapes=shapes)
    seqs = [torch.randn(n, D, generator=g) for n in (701, 5, 450)]
    refs = [P.input_convolution(s, w["c"].float().cpu()) for s in seqs]
    slots = [cache.alloc_slot() for _ in seqs]
    at = [0, 0, 0]
    for cuts in ([3, 2, 300], [398, 3, 150], [300, 0, 0]):
        members = [b for b in range(3) if cuts[b]]
        ctx, _ = build_context(cache, rt, [StepEntry(slots[b], [0] * cuts[b]) for b in members])
        y = torch.cat([seqs[b][at[b]:at[b] + cuts[b]] for b in members]).cuda()
        out = part.forward(y, cache.state.of(0, "block"), ctx, F32).cpu()
        ref = torch.cat([refs[b][at[b]:at[b] + cuts[b]] for b in members])
        assert float((out - ref).abs().max()) < 1e-5, (taps, cuts)
        for b in members:
            cache.commit(slots[b], cuts[b])
            at[b] += cuts[b]


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_update_normed_before_the_add_then_the_next_norm(dtype):
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(3)
    N, D, S = 7, 104, 3
    h, d = torch.randn(N, D, generator=g), torch.randn(S, N, D, generator=g)
    bias, wu, wn = torch.randn(D, generator=g), 1 + 0.1 * torch.randn(D, generator=g), torch.randn(D, generator=g)
    x = h + P.rms_norm(d.sum(0) + bias, wu, 1e-3)
    y = P.rms_norm(x, wn, 1e-5)
    hc = h.clone().cuda()
    got = K.postnorm_add_rmsnorm(hc, d.cuda(), bias.cuda(), wu.cuda(), 1e-3, wn.cuda(), 1e-5, dtype)
    close(hc, x, F32, "stream")
    close(got, y, dtype, "normed")
    rows = torch.tensor([5, 0], dtype=torch.int32).cuda()
    hc2 = h.clone().cuda()
    got = K.postnorm_add_rmsnorm(hc2, d.cuda(), None, wu.cuda(), 1e-3, wn.cuda(), 1e-5, F32, rows=rows, write_h=False)
    assert torch.equal(hc2.cpu(), h)
    close(got, P.rms_norm(h + P.rms_norm(d.sum(0), wu, 1e-3), wn, 1e-5)[[5, 0]], F32, "gathered rows")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_polynorm(dtype):
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(4)
    z = torch.randn(2, 5, 88, generator=g) * 1.5
    act = torch.tensor([0.6, -0.3, 0.25, 0.05])
    got = K.polynorm(z.cuda(), act.cuda(), 1e-4, dtype)
    close(got, P.polynorm(z.sum(0), act, 1e-4), dtype)


def attention_part(m, D, dtype, seed, edit=None):
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.parts import build_part
    cfg = config(8, D, 2048, 1.0, 1e-6, 1, [layer(m, None)])
    w = make_weights(cfg, seed)
    if edit is not None:
        edit(w)
    w = {k: v.cuda() for k, v in w.items()}
    spec = PartSpec("talking_attention", {
        "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "softmax_scale": m["scale"], "window": m["mask"]["size"],
        "keep_first": m["mask"]["keep_first"], "norm_eps": 1e-6}, prefix="l0.mix")
    return build_part("mixer", spec, w, runtime(dtype)), {k: v.float().cpu() for k, v in w.items()}


def run_mixer(mixer, rt, pieces):
    """Feeds one sequence's rows piece by piece through the mixer alone; returns all updates."""
    from lumenllm_b200.cache import KVCache
    from lumenllm_b200.engine.context import EntryView, StepEntry, build_context
    cache = KVCache({0: mixer.cache_need()}, 4096, 2, 4096, dtype=rt.dtype, device=rt.device)
    slot = cache.alloc_slot()
    outs = []
    for y in pieces:
        ctx, _ = build_context(cache, rt, [StepEntry(slot, [0] * y.shape[0])])
        out = mixer.forward(y.to(rt.dtype).cuda(), ctx, EntryView(ctx, 0, 0, True))
        outs.append((out.sum(0) if out.dim() == 3 else out).cpu())
        cache.commit(slot, y.shape[0])
    cache.check()
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", [attention(4, 2, 16, 24, 0.3, 9, 2), attention(6, 6, 32, 32, 0.11, 70, 0),
                               attention(3, 1, 32, 16, 0.2, 1000, 0), attention(2, 2, 64, 128, 0.15, 33, 70),
                               attention(5, 5, 24, 8, 0.5, 1, 1), attention(34, 1, 20, 10, 0.4, 50, 3),
                               attention(3, 3, 48, 80, 0.2, 70, 0)])
def test_talking_attention_part(m, dtype):
    """The mixer alone: a whole sequence, then the same continued token by token."""
    D, T = 48, 150
    mixer, w = attention_part(m, D, dtype, seed=5)
    y = torch.randn(T, D, generator=torch.Generator().manual_seed(6)).to(dtype).float()
    ref = P.talking_attention(y, w, "l0.mix.", m, 1e-6)
    got = run_mixer(mixer, runtime(dtype), [y[:131]] + [y[t:t + 1] for t in range(131, T)])
    close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_attention_in_passes_over_a_steps_rows(dtype, monkeypatch):
    """A step whose weights matrix would not fit its scratch is worked on in passes over its rows
    (here the scratch is made tiny: 64 rows a pass on the tensor cores, 7 in the general kernels);
    sequences and their 64-query tiles lie across the passes' borders."""
    from lumenllm_b200.ops import kernels as K
    m = attention(4, 2, 32, 32, 0.2, 90, 3)
    D = 48
    mixer, w = attention_part(m, D, dtype, seed=11)
    monkeypatch.setattr(K, "ATTN_TALK_PROMPT_SCRATCH_BYTES", 1)
    monkeypatch.setattr(K, "ATTN_TALK_SCRATCH_BYTES", 7 * 4 * 93 * 4)
    y = torch.randn(333, D, generator=torch.Generator().manual_seed(12)).to(dtype).float()
    ref = P.talking_attention(y, w, "l0.mix.", m, 1e-6)
    got = run_mixer(mixer, runtime(dtype), [y[:150], y[150:331], y[331:332], y[332:]])
    close(got, ref, dtype)


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_loud_key_at_every_edge_of_sight(dtype, decode):
    """Queries and values are the inputs themselves and keys the inputs shifted by seven channels,
    and one earlier token is made loud so that its KEY points where the last QUERY points (its own
    key then points elsewhere): this single key takes nearly all of the query's weight where it is in sight and none where it is not: far back among hundreds of
    keys, on both sides of the window's edge and of the kept first tokens' edge, and on both sides
    of page borders. Beside each case stands the mask that differs by one at that edge: the plain
    result under it must be far from the right one, else the case would show nothing."""
    H, d, D, T = 2, 32, 64, 300
    size, keep = 130, 3
    m = attention(H, H, d, d, 1.0, size, keep)

    def identity(w):
        for name in ("q", "k", "v"):
            w["l0.mix." + name] = torch.eye(D).to(BF16)
            w["l0.mix." + name + ".b"] = torch.zeros(D).to(BF16)
        w["l0.mix.k"] = torch.roll(torch.eye(D), 7, dims=0).to(BF16)
        w["l0.mix.q.norm"] = w["l0.mix.k.norm"] = torch.ones(D).to(BF16)
    mixer, w = attention_part(m, D, dtype, seed=7, edit=identity)
    g = torch.Generator().manual_seed(8)
    u = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
    query = T - 1
    lo = query - size + 1
    cases = [(0, None), (keep - 1, attention(H, H, d, d, 1.0, size, keep - 1)),
             (keep, attention(H, H, d, d, 1.0, size, keep + 1)), (63, None), (64, None),
             (lo - 1, attention(H, H, d, d, 1.0, size + 1, keep)), (lo, attention(H, H, d, d, 1.0, size - 1, keep)),
             (191, None), (192, None), (255, None), (256, None), (query - 1, None)]
    for loud, off_by_one in cases:
        y = torch.randn(T, D, generator=g) * 0.3
        y[loud] += 12 * torch.roll(u, -7)
        y[query] += 12 * u
        y = y.to(dtype).float()
        ref = P.talking_attention(y, w, "l0.mix.", m, 1e-6)
        if off_by_one is not None:
            wrong = P.talking_attention(y, w, "l0.mix.", off_by_one, 1e-6)
            assert float((wrong[query] - ref[query]).abs().max()) > 10 * tol(BF16) * max(1.0, float(ref.abs().max()))
        pieces = [y[:T - 40]] + [y[t:t + 1] for t in range(T - 40, T)] if decode else [y]
        got = run_mixer(mixer, runtime(dtype), pieces)
        close(got, ref, dtype, f"loud key {loud}")


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
        close(got, plain_logits(plain, name, toks), dtype, f"{name} {len(toks)} tokens")
    eng.check_kernels()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_residual_stream_after_every_layer(name, dtype, models, plain):
    """Layer by layer: the stream with each layer's last update added, against the plain one."""
    from lumenllm_b200.engine import StepEntry
    from lumenllm_b200.engine.context import EntryView
    from lumenllm_b200.ops import kernels as K
    cfg, w, _ = plain[name]
    toks = tokens_of(cfg, (45,), seed=2)[0]
    _, streams = P.forward(cfg, w, toks, streams=True)
    eng = engine_of(models, name, dtype)
    slot = eng.alloc_slot()
    ctx = eng.build_context([StepEntry(slot, toks)])
    h, pending = eng.model.embedding.forward(ctx.tokens, ctx), None
    for i, e in enumerate(eng.model.schedule):
        h, pending = eng.model.blocks[e.layer].forward(h, pending, ctx, EntryView(ctx, i, i, True))
        x = h.clone()
        K.postnorm_add_rmsnorm(x, pending.delta, pending.bias, pending.weight, pending.eps, None, 0.0, F32)
        close(x, streams[i], dtype, f"{name} after layer {i}")


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
        close(torch.cat(got), ref[:at], dtype, f"{name} cut as {cuts[:4]}...")
    eng.check_kernels()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_a_batch_of_unequal_requests_equals_each_alone(name, dtype, models, plain):
    """Prompts of unequal lengths in one step, then decoded together while the shorter requests
    leave; their slots and pages go to a second batch at once."""
    from lumenllm_b200.engine import StepEntry
    eng = engine_of(models, name, dtype, max_tokens=1024, max_slots=4)
    lens, tail = (1, 66, 140, 17), (3, 30, 12, 20)
    for round_ in range(2):
        seqs = tokens_of(SMALL[name], [n + t for n, t in zip(lens, tail)], seed=10 + round_)
        refs = [plain_logits(plain, name, s) for s in seqs]
        slots = [eng.alloc_slot() for _ in seqs]
        got = eng.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lens)])
        close(got, torch.cat([r[:n] for r, n in zip(refs, lens)]), dtype, f"{name} prompts")
        live = list(range(len(seqs)))
        for t in range(max(tail)):
            live = [b for b in live if t < tail[b]]
            got = eng.step([StepEntry(slots[b], [seqs[b][lens[b] + t]], [0]) for b in live])
            close(got, torch.stack([refs[b][lens[b] + t] for b in live]), dtype, f"{name} decode step {t}")
            for b in [b for b in live if t + 1 == tail[b]]:
                eng.free_slot(slots[b])
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


def test_windowed_layers_give_pages_back_and_keep_the_first(models, plain):
    """A long request under a short window holds few pages at a time, the page of its kept first
    tokens among them, and its logits stay right while pages go and come."""
    from lumenllm_b200.cache import PAGE
    from lumenllm_b200.engine import StepEntry
    name = "X"                                    # window 9, two kept tokens
    toks = tokens_of(SMALL[name], (3 * PAGE + 20,), seed=30)[0]
    ref = plain_logits(plain, name, toks)
    eng = engine_of(models, name, "float32", max_tokens=4 * PAGE, max_slots=2)
    slot = eng.alloc_slot()
    got = [eng.step([StepEntry(slot, toks[:PAGE + 5], list(range(PAGE + 5)))])]
    for t in range(PAGE + 5, len(toks)):
        got.append(eng.step([StepEntry(slot, [toks[t]], [0])]))
        g = eng.cache.groups[0]
        assert g.n_held[slot] <= 3 and g.table[slot, 0] != 0
    close(torch.cat(got), ref, "float32")
    other = eng.alloc_slot()                      # the pages given back serve another request meanwhile
    got = eng.step([StepEntry(other, toks[:2 * PAGE], [2 * PAGE - 1])])
    close(got, ref[2 * PAGE - 1:2 * PAGE], "float32")
    eng.free_slot(slot)
    eng.free_slot(other)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, models, plain):
    """build(EngineConfig).generate: batches, the scheduler's run-ahead and captured steps."""
    from lumenllm_b200 import EngineConfig, GenerateRequest, build
    name = "Z"
    cfg, w, _ = plain[name]
    built = build(EngineConfig(model_path=str(models[name]), dtype=dtype, context_size=512, max_batch=3))
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


def test_trace_replay_of_a_dabevik_model(models, plain, tmp_path):
    """bin/trace_run on a model of this design: prompt, portions and decoded tokens."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    name = "X"
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
