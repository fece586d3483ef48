"""The Volalorn design in the engine, on the CPU with the plain stand-in kernels and on the GPU
with the CUDA kernels (``-m gpu``): same bodies.

Everything is compared with ``plain_volalorn`` (float64, whole sequences, masks asked key by
key, one function per mechanism).  The configurations are made here; they differ from each
other in every size, in the order of the layers, in which options a mixer has (a stretched
rotation ladder or a plain one, a cap on the scores or none, first tokens kept or none) and in
whether a layer has a feed-forward; one has sizes that no vector width divides, one has windows,
chunks and head counts of 1.
"""

import copy

import pytest
import torch

import fake_kernels
import helpers
import plain_volalorn as plain
import replay
from shiso_llm_b200 import LLM, SamplingParams
from shiso_llm_b200.config import ConfigMissing, InvalidValue, VolalornConfig, plan_from_document
from shiso_llm_b200.parts import FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, BuildEnv, Model, PagedKV, PartSpec
from test_zetavik import BACKENDS, Feeder, backend_args, bind, build_env, close, dtypes, in_steps_and_batches, mixer_dtypes


def windowed(heads, kv_heads, dim, vdim, size, keep, rot_dims, base, scale):
    mask = {"size": size} if keep is None else {"size": size, "keep_first": keep}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": mask, "rot": {"dims": rot_dims, "base": base},
            "scale": scale}


def chunked(heads, kv_heads, dim, vdim, size, rot_dims, base, scale, softcap=None, scaling=None):
    doc = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size},
           "rot": {"dims": rot_dims, "base": base}, "scale": scale}
    if softcap is not None:
        doc["softcap"] = softcap
    if scaling is not None:
        doc["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return doc


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


DOC_A = {
    "architecture": "Volalorn", "vocab": 300, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
    "layers": [
        layer("attention_2", windowed(4, 2, 12, 8, 9, 3, 8, 1000.0, 0.3), 64),
        layer("attention", chunked(2, 1, 16, 16, 11, 16, 100.0, 0.25, 5.0, (4.0, 32, 8.0, 1.0)), 40),
        layer("attention_2", windowed(3, 3, 8, 10, 17, None, 4, 50.0, 0.5), None),
        layer("attention", chunked(4, 4, 8, 6, 5, 2, 7.0, 0.6), 24),
    ],
}

# windows, chunks, kept tokens and head counts of 1; more kept tokens than the window is wide; no logit scale
DOC_B = {
    "architecture": "Volalorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention", chunked(1, 1, 20, 36, 1, 20, 30.0, 0.2, 0.5), 96),
        layer("attention_2", windowed(2, 1, 16, 4, 1, 1, 16, 10000.0, 0.25), 32),
        layer("attention_2", windowed(6, 2, 8, 8, 6, 20, 6, 200.0, 0.4), None),
        layer("attention", chunked(3, 1, 12, 4, 64, 8, 500.0, 0.3, 30.0, (16.0, 16, 4.0, 0.5)), 48),
        layer("attention_2", windowed(1, 1, 24, 24, 40, 0, 2, 3.0, 0.2), 20),
    ],
}

# sizes that no vector width divides
DOC_C = {
    "architecture": "Volalorn", "vocab": 333, "width": 50, "norm": {"eps": 1e-5}, "logit_scale": 2.5,
    "layers": [
        layer("attention", chunked(3, 3, 6, 7, 13, 6, 11.0, 0.5, 2.0, (2.0, 20, 3.0, 1.5)), 22),
        layer("attention_2", windowed(6, 3, 10, 5, 7, 2, 2, 99.0, 0.35), 30),
        layer("attention_2", windowed(5, 1, 6, 9, 23, 5, 6, 17.0, 0.45), 14),
    ],
}

DOCS = {"A": (DOC_A, 3), "B": (DOC_B, 4), "C": (DOC_C, 5)}


def check_rows(got, ref, dtype, what):
    """Per-row error against the plain logits, relative to their spread.  float32: sums in another
    order and rsqrtf/expf/tanhf/sincosf stay below 1e-4 of the spread; bfloat16: matrices,
    activations and the cache rounded to 8 bits of mantissa through a few layers stay below a
    tenth.  A wrong key, page or window edge moves a row by far more."""
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    rms = (got - ref).pow(2).mean(-1).sqrt() / ref.std().item()
    bound = 1e-4 if dtype == "float32" else 0.1
    worst = int(rms.argmax())
    assert rms.max().item() <= bound, f"{what}: row {worst} differs by {rms.max().item():.3e} of the spread (> {bound})"


def reference_logits(doc, tensors, tokens):
    return plain.forward(doc, dict(tensors), tokens)


# --------------------------------------------------------------------------- configuration


def test_configuration_is_read_from_its_own_keys():
    arch, config, plan = plan_from_document(DOC_A)
    assert arch.name == "Volalorn" and isinstance(config, VolalornConfig)
    assert (config.vocab, config.width, config.eps, config.logit_scale) == (300, 48, 1e-5, 0.7)
    assert config.to_dict() == DOC_A and VolalornConfig.from_dict(config.to_dict()) == config
    assert all(l.mixer.kind == "masked_attention" and l.block.kind == "output_norm" for l in plan.layers)
    assert [l.mixer.params["mask"]["kind"] for l in plan.layers] == ["window", "chunk", "window", "chunk"]
    assert [l.mixer.params["weights"] for l in plan.layers] == ["softmax", "sigmoid", "softmax", "sigmoid"]
    assert [l.mixer.params["position"].kind for l in plan.layers] == ["rope_half_split", "rope_stretched", "rope_half_split", "rope_half_split"]
    assert plan.layers[2].mixer.params["mask"]["keep_first"] == 0 and plan.layers[3].mixer.params["softcap"] is None
    assert [l.feed_forward.kind if l.feed_forward else None for l in plan.layers] == ["polynorm_ff", "polynorm_ff", None, "polynorm_ff"]
    assert plan.head.params["tied_to"] is None and plan.final_norm.params["gain"] == 0.7
    assert VolalornConfig.from_dict(DOC_B).logit_scale == 1.0
    shapes = {s.name: s.shape for s in helpers.tensor_specs_of(DOC_A)}
    assert shapes["l0.norm1"] == () and shapes["final.norm"] == () and shapes["head"] == (300, 48)
    assert shapes["l0.mix.q"] == (48, 48) and shapes["l0.mix.k"] == (24, 48) and shapes["l0.mix.v"] == (16, 48)
    assert shapes["l0.mix.q.b"] == (48,) and shapes["l0.mix.v.b"] == (16,) and shapes["l0.mix.q.norm"] == (12,)
    assert shapes["l0.mix.o"] == (48, 32) and shapes["l0.mlp.act"] == (4,) and shapes["l0.mlp.up"] == (64, 48)
    assert shapes["l1.mix.pb"] == (2,) and shapes["l1.mix.g"] == (2, 48) and "l1.mix.q.b" not in shapes and "l0.mix.pb" not in shapes
    assert not any(n.startswith("l2.mlp") for n in shapes)


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

    with pytest.raises(ConfigMissing):
        VolalornConfig.from_dict(changed(("norm",), None))
    with pytest.raises(ConfigMissing):
        VolalornConfig.from_dict(changed(("layers", 0, "mixer", "vdim"), None))
    with pytest.raises(ConfigMissing):
        VolalornConfig.from_dict(changed(("layers", 1, "mixer", "rot", "scaling", "fast"), None))
    for path, value in [
        (("layers", 0, "type"), "attention_3"), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 7),
        (("layers", 0, "mixer", "rot", "dims"), 14), (("layers", 1, "mixer", "softcap"), 0.0), (("layers", 1, "mixer", "mask", "keep_first"), 2),
        (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.5), (("layers", 0, "mixer", "mask", "size"), 0),
        (("layers", 0, "mlp", "kind"), "glu"), (("vocab",), 0), (("layers",), []),
    ]:
        with pytest.raises(InvalidValue):
            VolalornConfig.from_dict(changed(path, value))


def test_cache_needs_windows_chunks_and_kept_tokens():
    _, _, plan = plan_from_document(DOC_A)
    env = BuildEnv(dtype=torch.float32, device=torch.device("cpu"), ops=fake_kernels)
    needs = Model(plan, env).cache_needs()
    assert needs[0] == PagedKV(2, 12, 9, 8, keep_first=3)
    assert needs[1] == PagedKV(1, 16, 11, 16)  # a chunk reaches no further back than its size
    assert needs[2] == PagedKV(3, 8, 17, 10) and needs[3] == PagedKV(4, 8, 5, 6)


def test_stretched_ladder_and_magnitude():
    env = BuildEnv(dtype=torch.float32, device=torch.device("cpu"), ops=fake_kernels)
    for rot in ({"dims": 16, "base": 100.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}},
                {"dims": 64, "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                {"dims": 6, "base": 11.0, "scaling": {"factor": 1.0, "original": 20, "fast": 3.0, "slow": 1.5}},
                {"dims": 8, "base": 500.0, "scaling": {"factor": 16.0, "original": 16, "fast": 4.0, "slow": 0.5}}):
        s = rot["scaling"]
        part = POSITION_ENCODINGS.build(PartSpec("rope_stretched", {"theta": rot["base"], "rotary_dim": rot["dims"], **s}), env, rot["dims"] + 2)
        want, magnitude = plain.frequencies(rot)
        inv_freq, dims = part.rotary()
        assert dims == rot["dims"] and abs(part.magnitude - magnitude) < 1e-12
        assert torch.allclose(inv_freq.double(), want, rtol=1e-6, atol=0)
    # the ladder's ends: a pair that turns often keeps its frequency, one that turns rarely is divided by the factor
    want, _ = plain.frequencies({"dims": 64, "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}})
    assert want[0] == 1.0 and abs(want[-1] * 40.0 / 10000.0 ** (-62 / 64) - 1.0) < 1e-12


# --------------------------------------------------------------------------- the whole model, every cut


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
def test_cuts_agree_with_each_other_far_more_closely(tmp_path, backend):
    """The same request whole, token by token and in portions: a row's keys are folded in runs
    counted from the start of its own lists, so cuts agree to rounding."""
    doc, seed = DOCS["A"]
    helpers.make_folder(tmp_path, doc, seed, std=0.15)
    toks = helpers.random_prompt(90, doc["vocab"], 77)
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=256, ctx=256, max_num_batched_tokens=256,
                                     **backend_args(backend))
        whole = replay.stack_rows(helpers.run_steps(engine, helpers.whole("a", toks)), "a", len(toks))
        single = replay.stack_rows(helpers.run_steps(engine, helpers.portions("b", toks, [1])), "b", len(toks))
        cut = replay.stack_rows(helpers.run_steps(engine, helpers.portions("c", toks, [5, 2, 31, 3])), "c", len(toks))
        bound = (1e-5 if dtype == "float32" else 0.05) * whole.std().item()
        assert (whole - single).abs().max().item() <= bound
        assert (whole - cut).abs().max().item() <= bound


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_with_a_request_that_joins(tmp_path, backend):
    """300 tokens one by one after a short prompt - every window and several chunks pass over
    decoded tokens - with a second request joining half-way; the trace runs twice in one engine,
    so every page and slot is used again, also the pages of the kept first tokens."""
    doc, seed = DOCS["B"]
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
    "architecture": "Volalorn", "vocab": 400, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
    "layers": [
        layer("attention_2", windowed(4, 2, 64, 64, 200, 10, 32, 10000.0, 0.125), 160),
        layer("attention", chunked(6, 2, 32, 48, 256, 32, 1000.0, 0.18, 15.0, (8.0, 128, 16.0, 1.0)), 96),
        layer("attention_2", windowed(2, 1, 128, 32, 77, 130, 64, 5000.0, 0.09), None),
        layer("attention", chunked(2, 2, 96, 128, 100, 48, 300.0, 0.1), 64),
        # heads of 64 rotated whole: single tokens take norm, rotation, store and attention in one launch
        layer("attention_2", windowed(4, 1, 64, 64, 130, 70, 64, 10000.0, 0.125), 96),
    ],
}


@pytest.mark.gpu
def test_long_portions_and_wide_heads(tmp_path):
    """Heads of real widths, a 700-token request: whole, in long and short portions, with a second
    request in the batch, and the last tokens decoded; windows and chunks longer than a tile of
    keys, cut at places no tile border meets."""
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


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_of_long_requests_through_the_trace_runner(tmp_path, dtype):
    """``bin/trace_run`` with heads of real widths and requests of hundreds of tokens: whole (the
    kernels for long portions), the last 40 tokens one by one (the kernels for single tokens, over
    windows and chunks that are full), long and short portions, and a mixed trace with portions up
    to 200 tokens beside single tokens, in a pool that the three requests fill."""
    doc = DOC_WIDE
    model_dir = tmp_path / "model"
    tensors = helpers.make_folder(model_dir, doc, 11, std=0.08)
    lengths = [700, 150, 300]
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab"], 80 + i) for i, n in enumerate(lengths)}
    steps, expect = [], []
    for rid, toks in requests.items():
        steps += helpers.whole(f"w-{rid}", toks)
        expect.append((f"w-{rid}", rid))
    steps += helpers.tail_one_by_one("t-r0", requests["r0"], 40)
    steps += helpers.portions("p-r0", requests["r0"], [300, 100, 258, 2, 1, 39])
    expect += [("t-r0", "r0"), ("p-r0", "r0")]
    steps += replay.mixed_trace({f"m-{k}": v for k, v in requests.items()}, 7, 1280, portion_sizes=(2, 5, 64, 130, 200))
    expect += [(f"m-{rid}", rid) for rid in requests]
    rows = replay.run_trace_run(model_dir, dtype, steps, 1280, tmp_path / "out", doc["vocab"])
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
            seq.append(int(reference_logits(doc, tensors, seq)[-1].argmax()))
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


def plan_layer(kind, mixer_doc, width, ff=None, eps=1e-5):
    """The layer's specs as the plan builder makes them, with tensors named ``l0.*``."""
    doc = {"architecture": "Volalorn", "vocab": 8, "width": width, "norm": {"eps": eps}, "layers": [layer(kind, mixer_doc, ff)]}
    return plan_from_document(doc)[2].layers[0]


WINDOW = windowed(6, 3, 10, 7, 12, 3, 6, 40.0, 0.4)
WINDOW_NO_KEEP = windowed(2, 2, 8, 8, 5, None, 8, 1000.0, 0.5)
CHUNK = chunked(4, 2, 12, 5, 9, 8, 60.0, 0.35, 3.0, (4.0, 24, 6.0, 1.0))
CHUNK_PLAIN = chunked(3, 1, 6, 10, 16, 4, 9.0, 0.7)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind,mixer_doc,fn", [
    ("attention_2", WINDOW, plain.window_softmax_attention), ("attention_2", WINDOW_NO_KEEP, plain.window_softmax_attention),
    ("attention", CHUNK, plain.chunk_sigmoid_attention), ("attention", CHUNK_PLAIN, plain.chunk_sigmoid_attention),
], ids=["window-keep", "window", "chunk-cap-stretch", "chunk"])
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


def planted_case(kind):
    """A mixer whose key matrix is its query matrix (and biases and norm weights alike), so that a
    row that repeats an earlier row's input scores ``scale * dim`` against it - far above the rest."""
    if kind == "attention_2":
        doc = windowed(2, 2, 16, 8, 50, 5, 4, 100.0, 1.0)
        same = {"l0.mix.k": "l0.mix.q", "l0.mix.k.b": "l0.mix.q.b", "l0.mix.k.norm": "l0.mix.q.norm"}
        # seen from row 299: [0, 5) and [250, 299]; pages of 4, runs of 32 keys from 0 and from 250
        places = (0, 3, 4, 5, 6, 31, 32, 150, 247, 248, 249, 250, 251, 252, 281, 282, 298)
        return doc, same, plain.window_softmax_attention, places, lambda j: j < 5 or j >= 250
    doc = chunked(2, 2, 16, 8, 64, 4, 100.0, 1.0, 25.0, (2.0, 64, 8.0, 1.0))
    # seen from row 299: [256, 299]
    places = (0, 63, 64, 191, 192, 254, 255, 256, 257, 260, 287, 288, 298)
    return doc, {"l0.mix.k": "l0.mix.q"}, plain.chunk_sigmoid_attention, places, lambda j: j >= 256


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", ["attention_2", "attention"])
def test_a_planted_key_at_the_edges_of_what_a_row_sees(backend, kind):
    """One key is made to stand out (the asking row repeats its input), so that whether it is seen
    decides the output: among the kept first tokens and right behind them, far back among hundreds,
    just outside and just inside the window or chunk, on either side of page borders and of the
    kernel's runs of 32 keys, and right before the asking row; the asking row comes at the end of a
    prompt's portion and as a decoded token."""
    dtype = torch.float32
    env = build_env(backend, dtype)
    doc, same, fn, places, seen = planted_case(kind)
    mixer = MIXERS.build(plan_layer(kind, doc, 32).mixer, env)
    specs = {s.name: s for s in mixer.tensor_specs()}
    from shiso_llm_b200.weights import random_tensors
    from shiso_llm_b200.weights.loader import target_dtype
    stored = random_tensors(list(specs.values()), 31, 0.3, "bfloat16", 0.1)
    for k_name, q_name in same.items():
        stored[k_name] = stored[q_name].clone()
    mixer.bind({k: v.to(env.device, target_dtype(specs[k], v.dtype, env.dtype)) for k, v in stored.items()})
    w = {k: v.double() for k, v in stored.items()}
    T = 300
    g = torch.Generator().manual_seed(3)
    base = torch.randn(T, 32, generator=g) * 0.1
    probe = torch.randn(32, generator=g)
    quiet = base.clone()
    quiet[T - 1] = probe * 1.5  # the asking row: the planted key's direction, another length (so another value row)
    without = fn(w, "l0.mix", doc, quiet.double(), 1e-5)[T - 1]
    for planted in places:
        h = quiet.clone()
        h[planted] = probe * 30.0  # (unit-RMS keys: the length goes into the value row only)
        want = fn(w, "l0.mix", doc, h.double(), 1e-5)
        moved = (want[T - 1] - without).abs().max().item() / without.abs().max().item()
        assert (moved > 0.02) == seen(planted), f"the plain implementation: a key planted at {planted} moves the last row by {moved:.2e}"
        for tail in (0, 40):
            feeder = Feeder(mixer, env, pages=128)
            got = [feeder.step([("a", h[: T - tail - 7])])["a"], feeder.step([("a", h[T - tail - 7 : T - tail])])["a"]]
            for t in range(T - tail, T):
                got.append(feeder.step([("a", h[t : t + 1])])["a"])
            close(torch.cat(got), want, dtype, f"{kind}: planted at {planted}, {tail} decoded", 4.0)


class SmallPoolFeeder(Feeder):
    """A pool of fewer pages than a sequence has positions for: tables are longer than the pool."""

    def __init__(self, mixer, env, pages, blocks, slots=3, page=4):
        from shiso_llm_b200.cache import CacheManager
        from shiso_llm_b200.engine.batch import StepBuilder
        self.mixer, self.env = mixer, env
        self.cache = CacheManager([mixer.cache_spec()], page, pages, slots, env.dtype, env.device, max_blocks_per_request=blocks)
        self.builder = StepBuilder(self.cache, env.device, 1024, slots)


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_first_tokens_and_pages_given_back_while_a_window_moves(backend):
    """A window of 6 over pages of 4 with two kept tokens: while 60 tokens are decoded the window
    group gives its pages back one by one and keeps the first; a second sequence takes them up.
    Every row of both is compared, the first rows (one key, two keys, ...) among them."""
    doc = windowed(2, 1, 8, 6, 6, 2, 8, 20.0, 0.5)
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        mixer = MIXERS.build(plan_layer("attention_2", doc, 24).mixer, env)
        w = bind(mixer, env, 7, 0.3)
        g = torch.Generator().manual_seed(4)
        a, b = torch.randn(70, 24, generator=g).to(dtype), torch.randn(50, 24, generator=g).to(dtype)
        want_a = plain.window_softmax_attention(w, "l0.mix", doc, a.double(), 1e-5)
        want_b = plain.window_softmax_attention(w, "l0.mix", doc, b.double(), 1e-5)
        feeder = SmallPoolFeeder(mixer, env, 12, 20)  # 70 + 50 positions would need 31 pages
        got_a, got_b = [], []
        for t in range(3):
            got_a.append(feeder.step([("a", a[t : t + 1])])["a"])
        got_a.append(feeder.step([("a", a[3:10])])["a"])
        for t in range(10, 70):
            parts = [("a", a[t : t + 1])]
            if t == 20:
                parts.append(("b", b[:2]))
            elif 20 < t <= 68:
                parts.insert(0, ("b", b[t - 19 : t - 18]))
            out = feeder.step(parts)
            got_a.append(out["a"])
            if "b" in out:
                got_b.append(out["b"])
        close(torch.cat(got_a), want_a, dtype, f"a moving window {dtype}", 4.0)
        close(torch.cat(got_b), want_b, dtype, f"the sequence that took its pages up {dtype}", 4.0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_polynomial_feed_forward_alone(backend):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        for width, ff, seed in ((36, 50, 17), (20, 7, 18), (64, 1024, 19)):
            part = FEED_FORWARDS.build(plan_layer("attention", CHUNK, width, ff).feed_forward, env)
            w = bind(part, env, seed, 0.3)
            g = torch.Generator().manual_seed(2)
            for rows in (1, 5, 70):
                h = torch.randn(rows, width, generator=g).to(dtype)
                want = plain.dense_ff(w, "l0.mlp", h.double(), 1e-5)
                y = part.forward(h.to(env.device), None)
                y = (y.materialize() if hasattr(y, "materialize") else y).double().cpu()
                close(y, want, dtype, f"polynomial feed-forward {width}x{ff}, {rows} rows {dtype}", 4.0)


def test_the_polynomial_activation_term_by_term():
    """Each coefficient alone: the unit-RMS first, second and third power, and the constant."""
    g = torch.Generator().manual_seed(5)
    z = torch.randn(4, 30, generator=g, dtype=torch.float64) * 2
    for i, power in enumerate((1, 2, 3)):
        c = torch.zeros(4, dtype=torch.float64)
        c[i] = 1.5
        u = z ** power
        want = 1.5 * u / torch.sqrt((u * u).mean(-1, keepdim=True) + 1e-5)
        assert torch.allclose(plain.poly_norm(z, c, 1e-5), want, rtol=1e-12)
        assert torch.allclose(fake_kernels.polynorm(z.float(), c.float(), 1e-5, torch.float32).double(), want, rtol=1e-5, atol=1e-6)
    c = torch.tensor([0.0, 0.0, 0.0, -0.25], dtype=torch.float64)
    assert torch.allclose(plain.poly_norm(z, c, 1e-5), torch.full_like(z, -0.25))


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_norm_of_an_output_added_to_the_stream(backend):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        for size in (50, 64, 3000):
            norm = NORMS.build(PartSpec("rmsnorm", {"tensor": "n", "size": size, "eps": 1e-5, "scalar": True, "gain": 0.5}), env)
            w = bind(norm, env, 3)
            assert w["n"].shape == ()
            g = torch.Generator().manual_seed(6)
            x = (torch.randn(9, size, generator=g) * 3 + 2).to(env.device)
            y = (torch.randn(9, size, generator=g) * 5).to(env.device, dtype)
            want = x.double().cpu() + plain.scalar_norm(y.double().cpu(), w["n"] * 0.5, 1e-5)
            residual = x.clone()
            rows = norm.add_normed(residual, y)
            assert rows.dtype == dtype
            close(residual.double().cpu(), want, torch.float32, f"residual + norm of an output, {size}")
            close(rows.double().cpu(), want, dtype, f"the new rows in the compute type, {size}")
