"""The Povilorn design in the engine, on the CPU with the plain stand-in kernels and on the GPU
with the CUDA kernels (``-m gpu``): same bodies.

Everything is compared with ``plain_povilorn`` (float64, whole sequences, one function per
mechanism).  The configurations are made here; they differ from each other in every size, in
the order of the layers and in which options they have: a looped stretch that starts at the
first layer, behind it, covers every layer, runs once, or is absent; a rotation over the whole
rotated part or over less of it, stretched or not; identity experts or none; one group or
several, all kept or few; a shared expert or none; a layer without feed-forward; key/value
heads of 1 and as many as query heads; a query temperature that steps at every position, once
in the test's lengths, or never; sizes that no vector width divides.
"""

import copy
import math

import pytest
import torch

import fake_kernels
import helpers
import plain_povilorn as plain
import replay
from shiso_llm_b200 import LLM, SamplingParams
from shiso_llm_b200.config import ConfigMissing, InvalidValue, PovilornConfig, plan_from_document
from shiso_llm_b200.parts import FEED_FORWARDS, MIXERS, NORMS, BuildEnv, Model, PagedKV, PartSpec
from test_zetavik import (BACKENDS, Feeder, Reference, backend_args, bind, build_env, check_rows, close, dtypes,
                          in_steps_and_batches, mixer_dtypes)


def attention(heads, kv_heads, dim, scale, coef=None, every=None):
    doc = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if coef is not None:
        doc["q_temp"] = {"coef": coef, "every": every}
    return doc


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, rot_dims, base, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}


def moe(experts, identity, top, count, keep, ff, limit, shared=None):
    doc = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}
    if count is not None:
        doc["router"]["groups"] = {"count": count, "keep": keep}
    if shared is not None:
        doc["shared"] = {"ff": shared[0], "limit": shared[1]}
    return doc


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# a stretch of two layers behind the first, three passes; identity experts and groups
DOC_A = {
    "architecture": "Povilorn", "vocab": 300, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        layer("latent_attention", latent(3, 8, 4, 6, 20, 0.3, 4, 50.0, (4.0, 32, 8.0, 1.0)), dense(64)),
        layer("attention", attention(4, 2, 12, 0.3, 0.5, 7), moe(6, 3, 3, 3, 2, 16, 0.8, (24, 1.2))),
        layer("latent_attention", latent(2, 4, 8, 10, 24, 0.2, 6, 100.0), None),
        layer("attention", attention(2, 2, 8, 0.4, 0.25, 1), dense(40)),
    ],
}

# no stretch at all; heads of 1; one group; no identity experts; no shared expert; no temperature; no embedding scale
DOC_B = {
    "architecture": "Povilorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention", attention(1, 1, 20, 0.2), moe(4, 0, 1, None, None, 24, 2.0)),
        layer("latent_attention", latent(1, 16, 8, 16, 32, 0.25, 8, 10000.0, (16.0, 16, 4.0, 0.5)), None),
        layer("attention", attention(6, 1, 8, 0.35, 1.5, 1000), dense(96)),
        layer("latent_attention", latent(5, 6, 2, 7, 12, 0.5, 2, 7.0), moe(5, 1, 6, 3, 3, 10, 0.5, (8, 0.25))),
    ],
}

# every layer inside the stretch, from the first on; sizes that no vector width divides; every router output chosen in one layer
DOC_C = {
    "architecture": "Povilorn", "vocab": 333, "width": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        layer("attention", attention(3, 3, 6, 0.5, 0.1, 13), dense(22)),
        layer("latent_attention", latent(3, 6, 10, 5, 11, 0.45, 6, 17.0, (2.0, 20, 3.0, 1.5)), moe(7, 2, 2, 1, 1, 6, 1.5, (14, 3.0))),
        layer("attention", attention(6, 2, 10, 0.35), moe(3, 1, 4, 2, 2, 9, 1.0)),
    ],
}

# a stretch that runs once (its vector is still added), over the last layers
DOC_D = {
    "architecture": "Povilorn", "vocab": 128, "width": 32, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.5},
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        layer("attention", attention(2, 1, 8, 0.3, 0.3, 5), None),
        layer("latent_attention", latent(2, 8, 4, 4, 8, 0.3, 4, 20.0), dense(16)),
    ],
}

DOCS = {"A": (DOC_A, 3), "B": (DOC_B, 4), "C": (DOC_C, 5), "D": (DOC_D, 6)}


def reference_logits(doc, tensors, tokens):
    margins = []
    logits = plain.forward(doc, dict(tensors), tokens, margins=margins)
    out = logits.as_subclass(Reference)
    out.margin = torch.stack(margins).min(0).values if margins else None
    return out


# --------------------------------------------------------------------------- configuration


def test_configuration_is_read_from_its_own_keys():
    arch, config, plan = plan_from_document(DOC_A)
    assert arch.name == "Povilorn" and isinstance(config, PovilornConfig)
    assert (config.vocab, config.width, config.eps, config.embedding_scale, config.loop) == (300, 48, 1e-5, 2.0, (1, 3, 3))
    assert config.to_dict() == DOC_A and PovilornConfig.from_dict(config.to_dict()) == config
    assert [l.mixer.kind for l in plan.layers] == ["latent_attention", "masked_attention", "latent_attention", "masked_attention"]
    assert all(l.block.kind == "pre_norm" and l.mixer_norm.kind == "dyt" for l in plan.layers) and plan.final_norm.kind == "dyt"
    # the run order: layer 0, then layers 1 and 2 three times, then layer 3; a pass begins with its vector, later ones with the embedding too
    assert [(e.layer, e.add_first, e.add_vector) for e in plan.order] == [
        (0, False, None), (1, False, ("loop.step", 0)), (2, False, None), (1, True, ("loop.step", 1)), (2, False, None),
        (1, True, ("loop.step", 2)), (2, False, None), (3, False, None)]
    m = plan.layers[1].mixer.params
    assert (m["mask"], m["values"], m["head_norm"], m["gate_per"], m["q_temperature"]) == ({"kind": "causal"}, "keys", "joined", "element", {"coef": 0.5, "every": 7})
    p = plan.layers[0].mixer.params
    assert p["q_rank"] is None and p["gate"] is None and p["position"].kind == "rope_stretched" and p["position"].params["interleaved"]
    assert plan.layers[2].mixer.params["position"].kind == "rope_half_split" and plan.layers[2].mixer.params["position"].params["rotary_dim"] == 6
    f = plan.layers[1].feed_forward.params
    assert (f["experts"], f["identity"], f["top"], f["group_count"], f["group_keep"], f["renormalize"], f["activation"], f["limit"]) == (9, 3, 3, 3, 2, True, "swish_clamped", 0.8)
    assert f["shared"].params["limit"] == 1.2 and f["shared_gate"] == "l1.mlp.shared.sg" and len(f["expert_names"]) == 6
    assert plan.layers[0].feed_forward.params["activation"] == "gelu_tanh" and plan.layers[2].feed_forward is None
    assert plan.embedding.params["scale"] == 2.0 and plan.head.params["tied_to"] is None
    shapes = {s.name: s.shape for s in helpers.tensor_specs_of(DOC_A)}
    assert shapes["loop.step"] == (3, 48) and shapes["l0.norm1.alpha"] == () and shapes["final.norm.b"] == (48,) and shapes["head"] == (300, 48)
    assert shapes["l1.mix.q"] == (48, 48) and shapes["l1.mix.k"] == (24, 48) and shapes["l1.mix.q.norm"] == (48,) and shapes["l1.mix.k.norm"] == (24,)
    assert shapes["l1.mix.g"] == (48, 48) and shapes["l1.mix.k.b"] == (24,) and "l1.mix.v" not in shapes
    assert shapes["l0.mix.q"] == (36, 48) and shapes["l0.mix.dkv"] == (24, 48) and shapes["l0.mix.uk"] == (24, 20) and shapes["l0.mix.uv"] == (18, 20)
    assert shapes["l1.mlp.router"] == (9, 48) and shapes["l1.mlp.correction"] == (9,) and shapes["l1.mlp.shared.sg"] == (1, 48)
    assert "l1.mlp.e5.gate" in shapes and "l1.mlp.e6.gate" not in shapes and not any(n.startswith("l2.mlp") or n.startswith("l2.norm2") for n in shapes)
    # no stretch: every layer once, no vectors
    _, config_b, plan_b = plan_from_document(DOC_B)
    assert config_b.loop is None and config_b.embedding_scale == 1.0 and "loop.step" not in {s.name for s in helpers.tensor_specs_of(DOC_B)}
    assert [(e.layer, e.add_first, e.add_vector) for e in plan_b.order] == [(i, False, None) for i in range(4)]
    assert plan_b.layers[0].mixer.params["q_temperature"] is None and plan_b.layers[0].feed_forward.params["shared"] is None
    assert [e.add_vector for e in plan_from_document(DOC_D)[2].order] == [None, ("loop.step", 0)]
    # a stretch without layers: nothing repeats, nothing is added, and a file may still hold the vectors
    empty = copy.deepcopy(DOC_D)
    empty["loop"] = {"start": 1, "stop": 1, "times": 3}
    plan_e = plan_from_document(empty)[2]
    assert [(e.layer, e.add_first, e.add_vector) for e in plan_e.order] == [(0, False, None), (1, False, None)] and "loop.step" in plan_e.unused_tensors


def test_configuration_refusals():
    def changed(path, value):
        doc = copy.deepcopy(DOC_A)
        at = doc
        for key in path[:-1]:
            at = at[key]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        return doc

    for path in [("norm",), ("layers", 1, "mixer", "kv_heads"), ("layers", 0, "mixer", "rot", "scaling", "slow"), ("layers", 1, "mlp", "expert", "limit"),
                 ("layers", 1, "mlp", "shared", "limit"), ("layers", 0, "mixer", "kv_rank"), ("loop", "times")]:
        with pytest.raises(ConfigMissing):
            PovilornConfig.from_dict(changed(path, None))
    for path, value in [
        (("layers", 0, "type"), "attention_2"), (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 1, "mixer", "vdim"), 8),
        (("layers", 0, "mixer", "rot", "dims"), 3), (("layers", 0, "mixer", "rot", "dims"), 6), (("layers", 1, "mixer", "q_temp", "every"), 0),
        (("layers", 1, "mlp", "router", "top"), 10), (("layers", 1, "mlp", "router", "groups", "count"), 4),
        (("layers", 1, "mlp", "router", "groups", "keep"), 4), (("layers", 1, "mlp", "expert", "limit"), 0.0),
        (("layers", 0, "mlp", "kind"), "glu"), (("loop", "stop"), 5), (("loop", "start"), 4), (("vocab",), 0), (("layers",), []),
    ]:
        with pytest.raises(InvalidValue):
            PovilornConfig.from_dict(changed(path, value))


def test_cache_needs():
    _, _, plan = plan_from_document(DOC_A)
    env = BuildEnv(dtype=torch.float32, device=torch.device("cpu"), ops=fake_kernels)
    needs = Model(plan, env).cache_needs()
    assert len(needs) == 8  # a cache of its own for every pass of a repeated layer
    assert needs[0] == PagedKV(1, 24, None, 0)  # one row [latent | rotated key part] per position, no value rows
    assert needs[1] == needs[3] == needs[5] == PagedKV(2, 12, None, 12)  # everything is kept: no window
    assert needs[2] == PagedKV(1, 32, None, 0) and needs[7] == PagedKV(2, 8, None, 8)


# --------------------------------------------------------------------------- the whole model, every cut


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cut_matches_the_plain_implementation(tmp_path, backend, name):
    doc, seed = DOCS[name]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    lengths = [70, 40, 7, 33, 1]
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab"], 20 + i) for i, n in enumerate(lengths)}
    reference = {rid: reference_logits(doc, tensors, toks) for rid, toks in requests.items()}
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=4, kv_cache_tokens=192, ctx=128,
                                     max_num_batched_tokens=128, **backend_args(backend))
        free = list(engine.cache.free_pages())
        steps, expect = [], []
        for rid, toks in requests.items():
            steps += helpers.whole(f"w-{rid}", toks)
            expect.append((f"w-{rid}", rid))
        steps += helpers.tail_one_by_one("t-r0", requests["r0"], 40)
        steps += helpers.portions("p-r0", requests["r0"], [13, 2, 7, 1, 3])
        steps += helpers.portions("p-r1", requests["r1"], [5, 4, 1])
        steps += helpers.portions("p-r3", requests["r3"], [2])
        expect += [("t-r0", "r0"), ("p-r0", "r0"), ("p-r1", "r1"), ("p-r3", "r3")]
        steps += replay.mixed_trace({f"m-{k}": v for k, v in requests.items()}, 3, 192)
        expect += [(f"m-{rid}", rid) for rid in requests]
        steps += replay.mixed_trace({f"n-{k}": v for k, v in reversed(list(requests.items()))}, 8, 192, tail=3)
        expect += [(f"n-{rid}", rid) for rid in requests]
        rows = helpers.run_steps(engine, steps)  # (checks the cache's books after every step)
        for trace_id, rid in expect:
            got = replay.stack_rows(rows, trace_id, len(requests[rid]))
            check_rows(got, reference[rid], dtype, f"{name} {dtype} {trace_id}")
        assert list(engine.cache.free_pages()) == free and engine.cache.slots.free_slots == 4


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_residual_stream_after_every_layer_run(tmp_path, backend):
    """The stream after every run of a layer (a repeated layer counts each time), before what the
    next pass adds: a vector or the embedding's rows added at the wrong place, or twice, shows here."""
    doc, seed = DOCS["A"]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    toks = helpers.random_prompt(19, doc["vocab"], 9)
    want = []
    plain.forward(doc, dict(tensors), toks, after_layer=lambda run, x: want.append(x.clone()))
    from shiso_llm_b200.engine import StepEntry
    from shiso_llm_b200.parts.model import stream_value
    engine = helpers.make_engine(tmp_path, "float32", page_size=4, kv_cache_tokens=64, ctx=64, max_num_batched_tokens=64, **backend_args(backend))
    got = {}
    engine.layer_hook = lambda pos, stream: got.__setitem__(pos, stream_value(stream).double().cpu())
    engine.step([StepEntry("a", toks, [len(toks) - 1])])
    assert sorted(got) == list(range(-1, len(want)))
    for run, x in enumerate(want):
        err = (got[run] - x).abs().max().item()
        assert err <= 2e-5 * x.abs().max().item(), f"after layer run {run}: {err:.3e}"


@pytest.mark.parametrize("backend", BACKENDS)
def test_cuts_agree_with_each_other_far_more_closely(tmp_path, backend):
    doc, seed = DOCS["C"]
    helpers.make_folder(tmp_path, doc, seed, std=0.15)
    toks = helpers.random_prompt(90, doc["vocab"], 77)
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=256, ctx=256, max_num_batched_tokens=256,
                                     **backend_args(backend))
        whole = replay.stack_rows(helpers.run_steps(engine, helpers.whole("a", toks)), "a", len(toks))
        single = replay.stack_rows(helpers.run_steps(engine, helpers.portions("b", toks, [1])), "b", len(toks))
        cut = replay.stack_rows(helpers.run_steps(engine, helpers.portions("c", toks, [5, 2, 31, 3])), "c", len(toks))
        bound = (1e-5 if dtype == "float32" else 0.1) * whole.std().item()
        # (bfloat16: a router's close call may fall otherwise in another cut; the rows before the first such call agree)
        if dtype == "float32":
            assert (whole - single).abs().max().item() <= bound
            assert (whole - cut).abs().max().item() <= bound
        else:
            assert (whole - single).abs().median().item() <= bound and (whole - cut).abs().median().item() <= bound


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_with_a_request_that_joins(tmp_path, backend):
    """300 tokens one by one after a short prompt - the query temperature steps many times over
    decoded tokens - with a second request joining half-way; the trace runs twice in one engine,
    so every page and slot is used again."""
    doc, seed = DOCS["A"]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    a = helpers.random_prompt(330, doc["vocab"], 5)
    b = helpers.random_prompt(110, doc["vocab"], 6)
    reference = {"a": reference_logits(doc, tensors, a), "b": reference_logits(doc, tensors, b)}
    steps = [([("a", a[:30], list(range(30)))], [])]
    for i in range(30, 330):
        entries = [("a", [a[i]], [0])]
        j = i - 130  # b: a prompt of 20 at a's position 130, then one token a step
        if j == 0:
            entries.insert(0, ("b", b[:20], list(range(20))))
        elif 0 < j <= 90:
            entries.append(("b", [b[19 + j]], [0]))
        steps.append((entries, [r for r, n in (("a", 329), ("b", 220)) if i == n]))
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=8, kv_cache_tokens=456, ctx=336, max_num_batched_tokens=64,
                                     **backend_args(backend))
        free = list(engine.cache.free_pages())
        helpers.run_steps(engine, steps[:150])
        engine.finish("a"), engine.finish("b")
        rows = helpers.run_steps(engine, steps)
        check_rows(replay.stack_rows(rows, "a", 330), reference["a"], dtype, f"long decoding {dtype}")
        check_rows(replay.stack_rows(rows, "b", 110), reference["b"], dtype, f"the request that joined {dtype}")
        assert list(engine.cache.free_pages()) == free and engine.cache.slots.free_slots == 4


DOC_WIDE = {
    "architecture": "Povilorn", "vocab": 400, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        layer("attention", attention(4, 2, 64, 0.11, 0.2, 200), dense(160)),
        layer("latent_attention", latent(3, 32, 32, 48, 64, 0.11, 32, 10000.0, (6.0, 128, 16.0, 1.0)), moe(6, 2, 2, 4, 2, 64, 1.25, (80, 2.0))),
        layer("attention", attention(2, 1, 128, 0.09, 0.3, 300), None),
        layer("latent_attention", latent(2, 64, 16, 128, 96, 0.1, 8, 300.0), dense(96)),
    ],
}


@pytest.mark.gpu
def test_long_portions_and_wide_heads(tmp_path):
    """Heads of real widths, a 700-token request: whole, in long and short portions, with a second
    request in the batch, and the last tokens decoded (the kernels for long portions and the ones
    for single tokens at a long context)."""
    tensors = helpers.make_folder(tmp_path, DOC_WIDE, 9, std=0.08)
    a = helpers.random_prompt(700, DOC_WIDE["vocab"], 1)
    b = helpers.random_prompt(150, DOC_WIDE["vocab"], 2)
    reference = {"a": reference_logits(DOC_WIDE, tensors, a), "b": reference_logits(DOC_WIDE, tensors, b)}
    for dtype in ("bfloat16", "float32"):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=4096, ctx=2048, max_num_batched_tokens=1024)
        rows = helpers.run_steps(engine, helpers.whole("w", a))
        check_rows(replay.stack_rows(rows, "w", 700), reference["a"], dtype, f"one long portion {dtype}")
        rows = helpers.run_steps(engine, helpers.portions("p", a, [300, 100, 260, 1, 39]))
        check_rows(replay.stack_rows(rows, "p", 700), reference["a"], dtype, f"long and short portions {dtype}")
        rows = helpers.run_steps(engine, helpers.tail_one_by_one("t", a, 24))
        check_rows(replay.stack_rows(rows, "t", 700), reference["a"], dtype, f"decoded at a long context {dtype}")
        steps = [([("a", a[:400], list(range(400))), ("b", b[:5], list(range(5)))], []),
                 ([("b", b[5:6], [0]), ("a", a[400:], list(range(300)))], ["a"]),
                 ([("b", b[6:], list(range(144)))], ["b"])]
        rows = helpers.run_steps(engine, steps)
        check_rows(replay.stack_rows(rows, "a", 700), reference["a"], dtype, f"a long portion in a batch {dtype}")
        check_rows(replay.stack_rows(rows, "b", 150), reference["b"], dtype, f"its neighbour {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(tmp_path, dtype):
    """``bin/trace_run`` in a process of its own over a pool that holds barely the live requests:
    whole, last tokens one by one, changing portions and a mixed trace, against the plain logits."""
    doc, seed = DOCS["C"]
    model_dir = tmp_path / "model"
    tensors = helpers.make_folder(model_dir, doc, seed, std=0.15)
    lengths = [70, 100, 40, 7, 33, 1]
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab"], 60 + i) for i, n in enumerate(lengths)}
    steps, expect = [], []
    for rid, toks in requests.items():
        steps += helpers.whole(f"w-{rid}", toks)
        expect.append((f"w-{rid}", rid))
    steps += helpers.tail_one_by_one("t-r1", requests["r1"], 32)
    steps += helpers.portions("p-r1", requests["r1"], [13, 2, 7, 64, 3])
    steps += helpers.portions("p-r0", requests["r0"], [2, 3, 1, 2, 5, 1, 1, 17])
    expect += [("t-r1", "r1"), ("p-r1", "r1"), ("p-r0", "r0")]
    steps += replay.mixed_trace({f"m-{k}": v for k, v in requests.items()}, 5, 320)
    expect += [(f"m-{rid}", rid) for rid in requests]
    rows = replay.run_trace_run(model_dir, dtype, steps, 320, tmp_path / "out", doc["vocab"])
    for trace_id, rid in expect:
        got = replay.stack_rows(rows, trace_id, len(requests[rid]))
        check_rows(got, reference_logits(doc, tensors, requests[rid]), dtype, f"{dtype} {trace_id}")


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_scheduler(tmp_path, backend):
    doc, seed = DOCS["A"]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    prompts = [helpers.random_prompt(n, doc["vocab"], 40 + n) for n in (19, 3, 30)]
    new = 12

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(plain.forward(doc, dict(tensors), seq)[-1].argmax()))
        return seq[len(prompt):]

    want = [plain_greedy(p) for p in prompts]
    args = backend_args(backend)
    llm = LLM(str(tmp_path), dtype="float32", ctx=64, page_size=4, max_num_seqs=2, max_num_batched_tokens=16, prefill_chunk=7,
              ops=args["ops"], device=args["device"])
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=new, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.engine.cache.check()
    assert llm.engine.cache.slots.free_slots == 2


# --------------------------------------------------------------------------- mechanisms alone


def plan_layer(kind, mixer_doc, width, mlp=None, eps=1e-5):
    """The layer's specs as the plan builder makes them, with tensors named ``l0.*``."""
    doc = {"architecture": "Povilorn", "vocab": 8, "width": width, "norm": {"eps": eps}, "layers": [layer(kind, mixer_doc, mlp)]}
    return plan_from_document(doc)[2].layers[0]


ATTENTION = attention(6, 3, 10, 0.4, 0.7, 4)
ATTENTION_ONE_GROUP = attention(5, 1, 6, 0.5)
LATENT = latent(5, 6, 4, 7, 13, 0.4, 4, 50.0, (4.0, 24, 6.0, 1.0))
LATENT_PART_ROTATED = latent(2, 8, 10, 3, 9, 0.3, 6, 9.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind,mixer_doc,fn", [
    ("attention", ATTENTION, plain.attention), ("attention", ATTENTION_ONE_GROUP, plain.attention),
    ("latent_attention", LATENT, plain.latent_attention), ("latent_attention", LATENT_PART_ROTATED, plain.latent_attention),
], ids=["attention-temperature", "attention-one-kv-head", "latent-stretched", "latent-part-rotated"])
def test_each_mixer_alone_in_steps_and_batches(backend, kind, mixer_doc, fn):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        mixer = MIXERS.build(plan_layer(kind, mixer_doc, 40).mixer, env)
        w = bind(mixer, env, 11)
        g = torch.Generator().manual_seed(1)
        a, b = torch.randn(37, 40, generator=g).to(dtype), torch.randn(9, 40, generator=g).to(dtype)
        want_a = fn(w, "l0.mix", mixer_doc, a.double(), 1e-5)
        want_b = fn(w, "l0.mix", mixer_doc, b.double(), 1e-5)
        in_steps_and_batches(mixer, env, dtype, a, b, want_a, want_b, kind, 4.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
def test_a_planted_key_far_back_and_at_the_kernels_borders(backend, kind):
    """One key is made to stand out (the asking row points the same way), so that whether it is seen,
    and with the right value, decides the output: at the sequence's first positions, far back among
    hundreds, on either side of page borders, of the runs of 32 keys and of the shares of 256 keys the
    kernels work in, and right before the asking row; the asking row comes at the end of a prompt's
    portion and as a decoded token."""
    dtype = torch.float32
    env = build_env(backend, dtype)
    if kind == "attention":
        doc, fn = attention(2, 2, 16, 1.0, 0.3, 100), plain.attention
        mixer = MIXERS.build(plan_layer(kind, doc, 32).mixer, env)
        # the key matrix is the query matrix (biases and norm weights alike): a row that repeats an earlier row's direction scores high
        specs = {s.name: s for s in mixer.tensor_specs()}
        from shiso_llm_b200.weights import random_tensors
        from shiso_llm_b200.weights.loader import target_dtype
        stored = random_tensors(list(specs.values()), 31, 0.3, "bfloat16", 0.1)
        for k_name, q_name in {"l0.mix.k": "l0.mix.q", "l0.mix.k.b": "l0.mix.q.b", "l0.mix.k.norm": "l0.mix.q.norm"}.items():
            stored[k_name] = stored[q_name].clone()
        mixer.bind({k: v.to(env.device, target_dtype(specs[k], v.dtype, env.dtype)) for k, v in stored.items()})
        w = {k: v.double() for k, v in stored.items()}
    else:
        doc, fn = latent(2, 8, 4, 8, 16, 1.0, 4, 100.0, (2.0, 64, 8.0, 1.0)), plain.latent_attention
        mixer = MIXERS.build(plan_layer(kind, doc, 32).mixer, env)
        w = bind(mixer, env, 31, 0.3)
    T = 600
    g = torch.Generator().manual_seed(3)
    base = torch.randn(T, 32, generator=g) * 0.1
    probe = torch.randn(32, generator=g)
    quiet = base.clone()
    quiet[T - 1] = probe * 3.0
    without = fn(w, "l0.mix", doc, quiet.double(), 1e-5)[T - 1]
    for planted in (0, 1, 3, 4, 31, 32, 150, 255, 256, 257, 511, 512, 543, 544, 597, 598):
        h = quiet.clone()
        h[planted] = probe * (30.0 if kind == "attention" else 3.0)
        want = fn(w, "l0.mix", doc, h.double(), 1e-5)
        if kind == "attention":  # (the latent's key is normed too, but its score rides on random matrices; the plain rows are the test there)
            moved = (want[T - 1] - without).abs().max().item() / without.abs().max().item()
            assert moved > 0.02, f"the plain implementation: a key planted at {planted} moves the last row by {moved:.2e} only"
        for tail in (0, 40):
            feeder = Feeder(mixer, env, pages=256)
            got = [feeder.step([("a", h[: T - tail - 7])])["a"], feeder.step([("a", h[T - tail - 7 : T - tail])])["a"]]
            for t in range(T - tail, T):
                got.append(feeder.step([("a", h[t : t + 1])])["a"])
            close(torch.cat(got), want, dtype, f"{kind}: planted at {planted}, {tail} decoded", 4.0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_query_temperature_steps_where_it_should(backend):
    """Positions on either side of every step of ``floor((p + 1) / every)``, in a prompt's portion and
    as single rows: with one key per position and queries that all point the same way, the output
    depends on the position through the temperature alone."""
    dtype = torch.float32
    env = build_env(backend, dtype)
    doc = attention(2, 1, 8, 0.5, 2.0, 6)
    mixer = MIXERS.build(plan_layer("attention", doc, 24).mixer, env)
    w = bind(mixer, env, 5, 0.3)
    assert [round(float(v), 6) for v in plain.query_temperature(torch.tensor([0, 4, 5, 6, 10, 11, 12]), 2.0, 6)] == [
        round(1.0 + 2.0 * math.log(n), 6) for n in (1, 1, 2, 2, 2, 3, 3)]
    g = torch.Generator().manual_seed(2)
    h = torch.randn(40, 24, generator=g)
    want = plain.attention(w, "l0.mix", doc, h.double(), 1e-5)
    got = Feeder(mixer, env).step([("a", h)])["a"]
    close(got, want, dtype, "temperature in a portion", 2.0)
    feeder, rows = Feeder(mixer, env), []
    rows.append(feeder.step([("a", h[:3])])["a"])
    for t in range(3, 40):  # single rows across the steps at 5, 11, 17, ...
        rows.append(feeder.step([("a", h[t : t + 1])])["a"])
    close(torch.cat(rows), want, dtype, "temperature of single rows", 2.0)
    # the same rows at positions shifted by one see another temperature: a kernel that counted from 1, or used p / every, differs
    flat = copy.deepcopy(doc)
    flat["q_temp"]["coef"] = 0.0
    assert (plain.attention(w, "l0.mix", flat, h.double(), 1e-5)[5:] - want[5:]).abs().max().item() > 1e-3


@pytest.mark.parametrize("backend", BACKENDS)
def test_neighbour_pairs_on_a_stretched_ladder(backend):
    """The rotation kernels against the plain rotation: neighbouring pairs, a ladder blended between
    its own and the divided frequencies, a magnitude on cosine and sine, fewer rotated entries than
    the part is wide, and positions far beyond the original length."""
    from types import SimpleNamespace
    from shiso_llm_b200.parts import POSITION_ENCODINGS
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        for rot, width in (({"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}, 8),
                           ({"dims": 6, "base": 11.0}, 10), ({"dims": 2, "base": 5.0, "scaling": {"factor": 16.0, "original": 16, "fast": 4.0, "slow": 0.5}}, 3)):
            s = rot.get("scaling") or {}
            part = POSITION_ENCODINGS.build(PartSpec("rope_stretched" if s else "rope_half_split",
                                                     {"theta": rot["base"], "rotary_dim": rot["dims"], "interleaved": True, **s}), env, width)
            f, magnitude = plain.stretched_ladder(rot)
            inv_freq, dims = part.rotary()
            assert part.interleaved and dims == rot["dims"] and abs(part.magnitude - magnitude) < 1e-12
            assert torch.allclose(inv_freq.double().cpu(), f, rtol=1e-6, atol=0)
            g = torch.Generator().manual_seed(4)
            x = torch.randn(7, 3, width, generator=g).to(dtype)
            positions = torch.tensor([0, 1, 2, 31, 32, 500, 4097], dtype=torch.int32)
            want = plain.rotate_neighbours(x.double(), positions, rot)
            out = torch.zeros(7, 3, width, dtype=dtype, device=env.device)
            step = SimpleNamespace(positions=positions.to(env.device))
            env.ops.rotate_heads(x.to(env.device), out, inv_freq, dims, step, magnitude=part.magnitude, interleaved=True)
            close(out.double().cpu(), want, dtype, f"neighbour pairs over {rot['dims']} of {width}", 4.0)


def ff_part(mlp, width):
    return plan_layer("attention", attention(1, 1, 4, 0.5), width, mlp).feed_forward


MLPS = {
    "dense": dense(50),
    "identity-groups-shared": moe(7, 3, 3, 5, 3, 14, 0.8, (20, 1.2)),
    "plain": moe(7, 0, 2, None, None, 9, 5.0),
    "all-chosen": moe(4, 2, 6, 2, 2, 8, 0.3, (8, 0.1)),
    "one-of-one-group": moe(8, 0, 1, 8, 1, 12, 1.0),
    "mostly-identity": moe(1, 5, 2, 3, 1, 6, 1.0),
}


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", list(MLPS))
def test_feed_forwards_alone(backend, name):
    mlp = MLPS[name]
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        part = FEED_FORWARDS.build(ff_part(mlp, 36), env)
        w = bind(part, env, 17, 0.3)
        g = torch.Generator().manual_seed(2)
        for rows in (1, 5, 70):
            h = (torch.randn(rows, 36, generator=g) * 1.5).to(dtype)
            margins = []
            want = plain.dense_ff(w, "l0.mlp", h.double()) if mlp["kind"] == "dense" else plain.moe_ff(w, "l0.mlp", mlp, h.double(), margins)
            y = part.forward(h.to(env.device), None)
            y = (y.materialize() if hasattr(y, "materialize") else y).double().cpu()
            sure = torch.ones(rows, dtype=torch.bool) if not margins or dtype == torch.float32 else margins[0] > 0.02
            assert torch.isfinite(y).all()
            if sure.any():  # (bfloat16: a row whose choice of experts hung on a close call may choose otherwise)
                close(y[sure], want[sure], dtype, f"{name} feed-forward, {rows} rows {dtype}", 4.0)


def test_the_clamped_pair_term_by_term():
    """Gates above the limit stop growing, gates far below stay (they are not clamped from below),
    the other half is clamped on both sides and shifted by one."""
    g = torch.tensor([[-9.0, -0.5, 0.5, 0.75, 3.0]], dtype=torch.float64)
    u = torch.tensor([[4.0, -4.0, 0.25, -0.75, 0.0]], dtype=torch.float64)
    got = fake_kernels._glu(g, u, "swish_clamped", 0.75)
    gc = torch.tensor([-9.0, -0.5, 0.5, 0.75, 0.75], dtype=torch.float64)
    uc = torch.tensor([0.75, -0.75, 0.25, -0.75, 0.0], dtype=torch.float64)
    assert torch.allclose(got[0], gc * torch.sigmoid(1.702 * gc) * (uc + 1.0), rtol=1e-12)
    z = torch.linspace(-4, 4, 9, dtype=torch.float64)[None]
    assert torch.allclose(fake_kernels._glu(z, torch.ones_like(z), "gelu_tanh", 0.0), plain.gelu_tanh(z), rtol=1e-12)
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12


@pytest.mark.parametrize("backend", BACKENDS)
def test_routing_with_a_correction_on_made_up_scores(backend):
    """Scores and corrections chosen so that every rule matters: the correction changes which group
    and which expert wins but not the weights; a group that is not kept cannot be chosen although
    the kept groups' corrected scores are negative; the weights are renormalised over the chosen."""
    env = build_env(backend, torch.float32)
    ops = env.ops
    # groups of two: {0,1} {2,3} {4,5}; scores (softmax of these logits) fall from expert 0 to 5
    logits = torch.tensor([[3.0, 2.5, 2.0, 1.5, 1.0, 0.5], [0.0, 0.1, 0.2, 0.3, 0.4, 0.5]])
    scores = torch.softmax(logits.double(), -1)
    # (1) no correction: the two best groups are {0,1} and {2,3}
    ids, weights = ops.moe_route(logits.to(env.device), 2, 3, 2, 1.0, False, True)
    assert ids.cpu().tolist() == [[0, 1], [5, 4]]
    # (2) a correction that lifts the last group above all and pushes the first below zero
    correction = torch.tensor([-1.0, -1.0, -0.5, -0.9, 0.5, -0.95])
    ids, weights = ops.moe_route(logits.to(env.device), 3, 3, 2, 1.0, False, True, correction=correction.to(env.device), renorm_eps=1e-20)
    choice = scores + correction.double()
    # row 0: groups by best corrected score: {4,5} first, then {2,3}; {0,1} is out although 0 and 1 have the largest scores
    assert ids.cpu().tolist()[0] == [4, 2, 3] and all(v < 0 for v in choice[0, :4].tolist())
    picked = torch.gather(scores, 1, ids.cpu().long())
    assert torch.allclose(weights.cpu().double(), picked / picked.sum(-1, keepdim=True), rtol=1e-5)
    want = plain.route(choice, 3, 3, 2)
    assert sorted(ids.cpu().tolist()[0]) == want[0].nonzero().flatten().tolist() and sorted(ids.cpu().tolist()[1]) == want[1].nonzero().flatten().tolist()
    # (3) logits in a column range of wider rows, as the router's product leaves them beside the shared expert's gate
    wide = torch.cat([logits, torch.full((2, 1), 99.0)], dim=1).to(env.device)
    ids2, weights2 = ops.moe_route(wide[:, :6], 3, 3, 2, 1.0, False, True, correction=correction.to(env.device), renorm_eps=1e-20)
    assert torch.equal(ids2.cpu(), ids.cpu()) and torch.equal(weights2.cpu(), weights.cpu())


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_tanh_norm_and_what_it_adds(backend):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        for size in (50, 64, 3000):
            norm = NORMS.build(PartSpec("dyt", {"tensor": "n", "size": size}), env)
            w = bind(norm, env, 3)
            assert w["n.alpha"].shape == () and w["n.b"].shape == (size,)

            def squash(x):
                return torch.tanh(w["n.alpha"] * x) * w["n"] + w["n.b"]

            g = torch.Generator().manual_seed(6)
            x = (torch.randn(9, size, generator=g) * 3 + 1).to(env.device)
            d1, d2 = (torch.randn(9, size, generator=g).to(env.device, dtype) for _ in range(2))
            close(norm.apply(x.clone()).double().cpu(), squash(x.double().cpu()), dtype, f"tanh norm, {size}")
            total = x.double().cpu() + d1.double().cpu() + d2.double().cpu()
            residual = x.clone()
            got = norm.add_apply(residual, (d1, d2))
            close(got.double().cpu(), squash(total), dtype, "sum of two + tanh norm")
            assert (residual.double().cpu() - total).abs().max().item() <= 1e-5
            rows = torch.tensor([7, 2], dtype=torch.int32, device=env.device)
            residual = x.clone()
            got = norm.add_apply(residual, d1, rows)
            close(got.double().cpu(), squash((x.double().cpu() + d1.double().cpu())[[7, 2]]), dtype, "rows")
            assert torch.equal(residual, x)


@pytest.mark.parametrize("backend", BACKENDS)
def test_rows_and_a_vector_added_to_the_stream(backend):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        g = torch.Generator().manual_seed(8)
        for tokens, hidden in ((5, 50), (1, 64), (33, 130)):
            x = torch.randn(tokens, hidden, generator=g).to(env.device)
            first = torch.randn(tokens, hidden, generator=g).to(env.device)
            waiting = torch.randn(tokens, hidden, generator=g).to(env.device, dtype)
            vector = torch.randn(hidden, generator=g).to(env.device)
            want = x.double() + first.double() + waiting.double() + vector.double()
            kept = x.clone()
            out = env.ops.stream_add(x, (waiting, first), vector, in_place=False)
            assert torch.equal(x, kept) and out.data_ptr() != x.data_ptr()
            assert (out.double() - want).abs().max().item() <= 1e-5
            out = env.ops.stream_add(x, (waiting, first), vector)
            assert out.data_ptr() == x.data_ptr() and (x.double() - want).abs().max().item() <= 1e-5
            y = torch.randn(tokens, hidden, generator=g).to(env.device)
            assert torch.equal(env.ops.stream_add(y.clone(), (), None), y)


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_scaled_embedding(backend):
    env = build_env(backend, torch.bfloat16 if backend == "cuda" else torch.float32)
    g = torch.Generator().manual_seed(1)
    table = torch.randn(20, 24, generator=g).to(env.device, env.dtype)
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32, device=env.device)
    got = env.ops.embed(ids, table, scale=3.0)
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), table.float().cpu()[[3, 19, 0, 3]] * 3.0)  # exact: the product is formed in float32


@pytest.mark.gpu
def test_gated_pairs_in_the_products_epilogues():
    """Every route of a gate/up product (a handful of rows, up to 192, the persistent kernels on one
    SM and on pairs) with each gated pair against the plain one, at sizes with ragged last tiles."""
    env = build_env("cuda", torch.bfloat16)
    g = torch.Generator().manual_seed(12)
    for k, inter in ((256, 384), (200, 72), (1024, 1416)):
        w = (torch.randn(2 * inter, k, generator=g) * 0.08).to(env.device, torch.bfloat16)
        for rows in (1, 8, 9, 70, 192, 200, 511, 520, 1100):
            x = torch.randn(rows, k, generator=g).to(env.device, torch.bfloat16)
            for act, limit in (("gelu_tanh", 0.0), ("swish_clamped", 0.7), ("swish_clamped", 6.0), ("silu", 0.0)):
                got = env.ops.linear_glu(x, w, torch.bfloat16, act, limit).double().cpu()
                want = fake_kernels.linear_glu(x.cpu(), w.cpu(), torch.float64, act, limit)
                close(got, want, torch.bfloat16, f"{act} {limit}: {rows} x {2 * inter} x {k}")
        x = torch.randn(33, k, generator=g).to(env.device)
        got = env.ops.linear_glu(x, w.float(), torch.float32, "gelu_tanh", 0.0).double().cpu()
        close(got, fake_kernels.linear_glu(x.cpu(), w.float().cpu(), torch.float64, "gelu_tanh", 0.0), torch.float32, f"float32 gelu {k}")


@pytest.mark.gpu
def test_a_gate_per_entry_behind_the_fast_attention_kernels():
    """``gate_rows`` alone, on column ranges of wider rows, in both types and at widths no vector divides."""
    for dtype in (torch.float32, torch.bfloat16):
        env = build_env("cuda", dtype)
        g = torch.Generator().manual_seed(13)
        for tokens, cols, pad in ((5, 64, 0), (3, 50, 6), (70, 384, 128)):
            rows = torch.randn(tokens, cols + pad, generator=g).to(env.device, dtype)
            gates = torch.randn(tokens, cols + 2 * pad, generator=g).to(env.device, dtype)
            x, gate = rows[:, :cols], gates[:, pad : pad + cols]
            want = x.double().cpu() * torch.sigmoid(gate.double().cpu())
            untouched = rows[:, cols:].clone()
            got = env.ops.gate_rows(x, gate)
            close(got.double().cpu(), want, dtype, f"gate rows {tokens} x {cols}")
            assert torch.equal(rows[:, cols:], untouched)
