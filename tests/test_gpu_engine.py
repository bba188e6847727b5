"""The engine on a GPU against the plain implementation, in float32 and in bfloat16."""

import pytest
import torch

import plain_model
from helpers import BF16_TIE_GAP, CONFIGS, assert_close, bf16_weights, prompts_for, write_model

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def reference_weights(weights, dtype):
    return weights if dtype == "float32" else bf16_weights(weights)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        weights = plain_model.random_weights(cfg, seed=31 + len(name), matrix_std=0.06, norm_std=0.1)
        out[name] = (write_model(tmp_path_factory.mktemp(f"tiny_{name}"), cfg, weights), cfg, weights)
    return out


def make_engine(folder, dtype, max_tokens=2048, **kw):
    from dryft_flash_infer_b200 import Engine

    engine = Engine(folder, dtype=dtype, max_tokens=max_tokens, **kw)
    for group in engine.cache.groups:       # anything read beyond what was written shows as NaN
        group.k.fill_(float("nan"))
        group.v.fill_(float("nan"))
    return engine


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_each_request_alone_and_whole(folders, name, dtype):
    from dryft_flash_infer_b200 import StepEntry

    folder, cfg, weights = folders[name]
    engine = make_engine(folder, dtype)
    for prompt in prompts_for(cfg, [1, 2, 17, 64, 65, 150], seed=1):
        slot = engine.open_slot()
        logits = engine.step([StepEntry(slot, prompt, list(range(len(prompt))))])
        engine.close_slot(slot)
        assert_close(logits, plain_model.forward(cfg, reference_weights(weights, dtype), prompt), dtype,
                     f"prompt of {len(prompt)}")
    engine.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_last_32_tokens_one_by_one(folders, name, dtype):
    from dryft_flash_infer_b200 import StepEntry

    folder, cfg, weights = folders[name]
    engine = make_engine(folder, dtype)
    for prompt in prompts_for(cfg, [33, 100], seed=2):
        want = plain_model.forward(cfg, reference_weights(weights, dtype), prompt)
        slot = engine.open_slot()
        head = len(prompt) - 32
        first = engine.step([StepEntry(slot, prompt[:head], [head - 1])])
        rows = [first[0]]
        for t in range(head, len(prompt)):
            rows.append(engine.step([StepEntry(slot, [prompt[t]], [0])])[0])
        engine.close_slot(slot)
        assert_close(torch.stack(rows), want[head - 1:], dtype, f"decode after {head}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_one_after_another(folders, name, dtype):
    """Batches of unequal lengths; shorter requests end earlier; the next batch takes the
    freed slots and pages, which still hold the earlier batch's keys."""
    from dryft_flash_infer_b200 import StepEntry

    folder, cfg, weights = folders[name]
    engine = make_engine(folder, dtype, max_tokens=64 * 8)
    ref_w = reference_weights(weights, dtype)
    seen_slots = []
    for round_, lengths in enumerate([(5, 9, 17, 70), (23, 1, 4, 11), (66, 3)]):
        prompts = prompts_for(cfg, lengths, seed=10 + round_)
        decode = [3 + i for i in range(len(prompts))]          # the first request ends first
        full = [p + prompts_for(cfg, [d], seed=50 + i)[0] for i, (p, d) in enumerate(zip(prompts, decode))]
        want = [plain_model.forward(cfg, ref_w, seq) for seq in full]
        slots = [engine.open_slot() for _ in prompts]
        seen_slots.append(list(slots))
        logits = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        for i, p in enumerate(prompts):
            assert_close(logits[i], want[i][len(p) - 1], dtype, f"round {round_} prefill {i}")
        live = list(range(len(prompts)))
        for t in range(max(decode)):
            live = [i for i in live if t < decode[i]]
            logits = engine.step([StepEntry(slots[i], [full[i][len(prompts[i]) + t]], [0]) for i in live])
            for row, i in enumerate(live):
                assert_close(logits[row], want[i][len(prompts[i]) + t], dtype, f"round {round_} seq {i} step {t}")
            for i in live:
                if t + 1 == decode[i]:
                    engine.close_slot(slots[i])
        engine.cache.book.check()
        assert engine.cache.live_slots == 0
    assert seen_slots[1][0] == seen_slots[0][0]                  # slots are used again


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_the_first_tokens(folders, dtype):
    from dryft_flash_infer_b200 import StepEntry

    folder, cfg, weights = folders["B"]
    engine = make_engine(folder, dtype)
    seq = prompts_for(cfg, [200], seed=3)[0]
    want = plain_model.forward(cfg, reference_weights(weights, dtype), seq)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, [t], [0])])[0] for t in seq]     # from the very first token on
    engine.close_slot(slot)
    got = torch.stack(rows)
    assert_close(got[:4], want[:4], dtype, "first tokens")
    assert_close(got, want, dtype, "200 single-token steps")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunks_of_any_size_agree(folders, dtype):
    from dryft_flash_infer_b200 import StepEntry

    folder, cfg, weights = folders["A"]
    engine = make_engine(folder, dtype)
    seq = prompts_for(cfg, [131], seed=4)[0]
    want = plain_model.forward(cfg, reference_weights(weights, dtype), seq)
    slot = engine.open_slot()
    rows, at = [], 0
    for size in (1, 63, 1, 2, 64):
        piece = seq[at:at + size]
        rows.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]))
        at += size
    engine.close_slot(slot)
    assert at == len(seq)
    assert_close(torch.cat(rows), want, dtype, "chunked prompt")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds(tmp_path, dtype):
    """One key far back is made to stand out: the query of the last token is scaled so that it
    matches the key at position 3 much better than the other 400.  A kernel that drops, repeats or
    misplaces a page of keys gives other logits than the plain implementation."""
    from dryft_flash_infer_b200 import Engine, StepEntry

    cfg = dict(plain_model.TINY_B, num_hidden_layers=1)
    weights = plain_model.random_weights(cfg, seed=77, matrix_std=0.05)
    p = "model.layers.0.self_attn."
    weights[p + "q_norm.weight"] = weights[p + "q_norm.weight"] * 6.0    # sharp attention
    weights[p + "v_proj.weight"] = weights[p + "v_proj.weight"] * 4.0    # and values that matter
    seq = prompts_for(cfg, [401], seed=5)[0]
    seq[-1] = seq[3]                     # same token: same direction of q and k up to the rotation
    folder = write_model(tmp_path, cfg, weights)
    ref_w = reference_weights(weights, dtype)
    want = plain_model.forward(cfg, ref_w, seq)
    engine = Engine(folder, dtype=dtype, max_tokens=1024)
    slot = engine.open_slot()
    whole = engine.step([StepEntry(slot, seq, [len(seq) - 1])])
    engine.close_slot(slot)
    slot = engine.open_slot()
    engine.step([StepEntry(slot, seq[:-1], [])])
    single = engine.step([StepEntry(slot, seq[-1:], [0])])
    engine.close_slot(slot)
    assert_close(whole[0], want[-1], dtype, "far key, whole")
    assert_close(single[0], want[-1], dtype, "far key, decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from dryft_flash_infer_b200 import Engine

    folder, cfg, weights = folders[name]
    engine = Engine(folder, dtype=dtype)
    prompts = prompts_for(cfg, [5, 9, 17] if name == "A" else [1, 4, 11, 23], seed=6)
    steps = 8 if name == "A" else 12
    rows = list(engine.generate(prompts, steps))
    assert len(rows) == steps and all(len(r) == len(prompts) for r in rows)
    ref_w = reference_weights(weights, dtype)
    for i, prompt in enumerate(prompts):
        got = [r[i] for r in rows]
        if dtype == "float32":
            assert got == plain_model.greedy_continue(cfg, ref_w, prompt, steps)
        else:
            # bfloat16 may pick another token where two logits are close: follow the engine's own tokens
            seq = list(prompt)
            for token in got:
                logits = plain_model.forward(cfg, ref_w, seq)[-1]
                gap = float(logits.max() - logits[token])
                assert gap <= BF16_TIE_GAP, f"token {token} is {gap} below the best"
                seq.append(token)
    # a second call shares nothing with the first, and freed slots were all returned
    again = list(engine.generate(prompts, steps))
    assert again == rows and engine.cache.live_slots == 0
    assert list(engine.generate(prompts, 0)) == []
    with pytest.raises(ValueError):
        list(engine.generate(prompts, -1))


@pytest.mark.parametrize("dtype", DTYPES)
def test_temperature_sampling_does_not_depend_on_the_batch(folders, dtype):
    from dryft_flash_infer_b200 import Engine, Request

    folder, cfg, weights = folders["B"]
    engine = Engine(folder, dtype=dtype)
    prompts = prompts_for(cfg, [1, 4, 11, 23], seed=7)
    together = list(engine.generate(prompts, 12, temperature=0.8, seed=5))
    assert any(len({r[i] for r in together}) > 1 for i in range(4))
    requests = [Request(p, 12, request_id=i) for i, p in enumerate(prompts)]
    engine.generate_requests(requests, max_batch=1, temperature=0.8, seed=5)       # one batch after another
    if dtype == "float32":
        for i, r in enumerate(requests):
            assert r.output == [row[i] for row in together]
    # stop tokens end a sequence early
    stop = together[2][0]
    rows = list(engine.generate(prompts, 12, temperature=0.8, seed=5, stop_token_ids=(stop,)))
    assert rows[2][0] == stop and all(r[0] is None for r in rows[3:])
    assert engine.cache.live_slots == 0


def test_sampled_tokens_follow_the_distribution(folders):
    """Each sampled token lies where the inverse CDF of the plain softmax puts its uniform number."""
    from dryft_flash_infer_b200 import Engine
    from dryft_flash_infer_b200.sampling import uniform_for

    folder, cfg, weights = folders["B"]
    engine = Engine(folder, dtype="float32")
    prompt = prompts_for(cfg, [9], seed=8)[0]
    got = [r[0] for r in engine.generate([prompt], 10, temperature=0.8, seed=11)]
    seq = list(prompt)
    for step, token in enumerate(got):
        probs = plain_model.temperature_probabilities(plain_model.forward(cfg, weights, seq)[-1], 0.8)
        cdf = torch.cumsum(probs, 0)
        u = uniform_for(11, 0, step)
        low = float(cdf[token - 1]) if token else 0.0
        assert low - 1e-5 <= u <= float(cdf[token]) + 1e-5, f"step {step}: u={u} not in [{low}, {float(cdf[token])}]"
        seq.append(token)


def test_engine_errors_are_loud(folders):
    from dryft_flash_infer_b200 import Engine, StepEntry
    from dryft_flash_infer_b200.cache import CacheError

    folder, cfg, _ = folders["A"]
    engine = Engine(folder, dtype="float32", max_tokens=128)
    a, b = engine.open_slot(), engine.open_slot()
    with pytest.raises(CacheError, match="out of slots"):
        engine.open_slot()
    with pytest.raises(CacheError, match="out of cache pages"):
        engine.step([StepEntry(a, [1] * 65, []), StepEntry(b, [1] * 65, [])])
    with pytest.raises(ValueError, match="vocabulary"):
        engine.step([StepEntry(a, [cfg["vocab_size"]], [0])])
    with pytest.raises(ValueError, match="twice"):
        engine.step([StepEntry(a, [1], [0]), StepEntry(a, [2], [0])])
    with pytest.raises(ValueError, match="brings no tokens"):
        engine.step([StepEntry(a, [1], [0]), StepEntry(b, [], [-1])])
    with pytest.raises(ValueError, match="outside the 1 token"):
        engine.step([StepEntry(a, [1], [1])])
    engine.close_slot(a)
    with pytest.raises(CacheError, match="freed twice"):
        engine.close_slot(a)


QWEN3_4B_WIDTHS = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2560, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728, "vocab_size": 151936,
    "rope_theta": 5000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "hidden_act": "silu",
    "max_position_embeddings": 40960,
}


@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    """Two layers at the widths of Qwen3-4B with random weights, as a model folder, and the same
    weights as the plain implementation takes them (read back from the file, not from the engine)."""
    from dryft_flash_infer_b200.config import config_from_dict
    from dryft_flash_infer_b200.weights import ModelFiles, write_random_model

    folder = write_random_model(config_from_dict(QWEN3_4B_WIDTHS), 5, tmp_path_factory.mktemp("wide"), torch.bfloat16)
    files = ModelFiles(folder)
    weights = {name: files.tensor(name).float() for name in files.names()}
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 151936, (n,), generator=g).tolist() for n in (300, 64, 129, 7)]
    # the plain implementation on the CPU: the places of each prompt that the engine is asked for
    places = {0: [0, 150, 296, 297, 298, 299], 1: [0, 60, 61, 62, 63], 2: [0, 125, 126, 127, 128], 3: [0, 3, 4, 5, 6]}
    want = {i: plain_model.forward(QWEN3_4B_WIDTHS, weights, prompts[i], places=places[i]) for i in places}
    return folder, prompts, places, want


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_sizes_of_the_benchmark_model_against_the_plain_implementation(wide_model, dtype):
    """Two layers at the widths of Qwen3-4B (the sizes the tcgen05 kernels are built for) against the plain
    implementation on the CPU: a batch of four unequal prompts minus their last three tokens, those three
    one by one (the decode path on fixed buffers), the longest prompt whole and alone, and generation."""
    from dryft_flash_infer_b200 import Engine, StepEntry
    from dryft_flash_infer_b200.ops import kernels

    folder, prompts, places, want = wide_model
    engine = Engine(folder, dtype=dtype, max_tokens=2048)
    slots = [engine.open_slot() for _ in prompts]
    first = engine.step([StepEntry(s, p[:-3], [0, len(p) - 4]) for s, p in zip(slots, prompts)])
    for i, p in enumerate(prompts):
        assert_close(first[2 * i], want[i][0], dtype, f"prompt {i}, first place", family="wide")
        assert_close(first[2 * i + 1], want[i][-4], dtype, f"prompt {i}, place {len(p) - 4}", family="wide")
    for t in (3, 2, 1):
        rows = engine.step([StepEntry(s, [p[len(p) - t]], [0]) for s, p in zip(slots, prompts)])
        for i in range(len(prompts)):
            assert_close(rows[i], want[i][-t], dtype, f"prompt {i}, {t} from the end, one token", family="wide")
    for s in slots:
        engine.close_slot(s)
    slot = engine.open_slot()
    whole = engine.step([StepEntry(slot, prompts[0], [0, 150, 299])])
    engine.close_slot(slot)
    for row, index in enumerate((0, 1, 5)):
        assert_close(whole[row], want[0][index], dtype, f"whole prompt, place {places[0][index]}", family="wide")
    # generation (prompt step, then decode steps through the graph): the first token is the plain argmax
    tokens = [r[0] for r in engine.generate([prompts[1]], 3)]
    best = want[1][-1]
    assert float(best.max() - best[tokens[0]]) <= (0 if dtype == "float32" else 0.05)
    assert kernels.tc_error() == 0 and kernels.attention_tc_error(128) == 0
    engine.check_status()


TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 80, "num_attention_heads": 5,
    "num_key_value_heads": 5, "head_dim": 48, "intermediate_size": 72, "vocab_size": 100, "rope_theta": 500000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "hidden_act": "silu", "max_position_embeddings": 2048,
}


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_third_shape_and_a_batch_wider_than_the_skinny_kernels(tmp_path, dtype):
    """Head size 48 with as many key/value heads as query heads (another kernel path than 16/32/128), and a
    batch of 70 sequences, which is past what the decode kernels for small batches take."""
    from dryft_flash_infer_b200 import Engine, StepEntry

    cfg = TINY_C
    weights = plain_model.random_weights(cfg, seed=8, matrix_std=0.08, norm_std=0.1)
    folder = write_model(tmp_path, cfg, weights)
    ref_w = reference_weights(weights, dtype)
    engine = Engine(folder, dtype=dtype, max_tokens=70 * 128)
    prompts = prompts_for(cfg, [3 + (7 * i) % 40 for i in range(70)], seed=21)
    want = [plain_model.forward(cfg, ref_w, p) for p in prompts]
    slots = [engine.open_slot() for _ in prompts]
    logits = engine.step([StepEntry(s, p[:-2], [len(p) - 3]) for s, p in zip(slots, prompts)])
    for i, p in enumerate(prompts):
        assert_close(logits[i], want[i][len(p) - 3], dtype, f"prefill {i}")
    for t in (2, 1):
        logits = engine.step([StepEntry(s, [p[len(p) - t]], [0]) for s, p in zip(slots, prompts)])
        for i, p in enumerate(prompts):
            assert_close(logits[i], want[i][len(p) - t], dtype, f"decode {i} -{t}")
    for s in slots:
        engine.close_slot(s)
    # and through the generation loop (fixed buffers, CUDA graph) with all 70 at once
    rows = list(engine.generate(prompts, 3))
    assert len(rows) == 3 and all(len(r) == 70 for r in rows)
    if dtype == "float32":
        for i in (0, 33, 69):
            assert [r[i] for r in rows] == plain_model.greedy_continue(cfg, ref_w, prompts[i], 3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_large_tensors_load_through_pinned_pieces(tmp_path, dtype, monkeypatch):
    """Tensors of 4 MB or more are read by the native reader's threads into pinned memory piece by
    piece; with small pieces a tensor takes several, and every element still lands in its place."""
    from dryft_flash_infer_b200 import Engine
    from dryft_flash_infer_b200.config import config_from_dict
    from dryft_flash_infer_b200.weights import ModelFiles, loader, write_random_model

    raw = dict(plain_model.TINY_A, vocab_size=40000, intermediate_size=16384)      # embedding 5 MB, gate/up/down 2 MB each
    folder = write_random_model(config_from_dict(raw), 3, tmp_path / "wide", torch.bfloat16)
    monkeypatch.setattr(loader, "_STAGE_BYTES", 1 << 20)
    monkeypatch.setattr(loader, "_STAGED_FROM", 1 << 20)
    engine = Engine(str(folder), dtype=dtype, max_tokens=256)
    files = ModelFiles(folder)
    want = files.tensor("model.embed_tokens.weight").to(engine.model.embedding.dtype)
    assert torch.equal(engine.model.embedding.cpu(), want)
    ffn = engine.model.blocks[1].feed_forward
    gate_up = torch.cat([files.tensor("model.layers.1.mlp.gate_proj.weight"), files.tensor("model.layers.1.mlp.up_proj.weight")])
    assert torch.equal(ffn.gate_up.cpu(), gate_up.to(ffn.gate_up.dtype))
    assert torch.equal(ffn.down.cpu(), files.tensor("model.layers.1.mlp.down_proj.weight").to(ffn.down.dtype))


TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 136, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 264, "vocab_size": 211, "rope_theta": 20000.0,
    "rms_norm_eps": 2e-5, "tie_word_embeddings": True, "hidden_act": "silu", "max_position_embeddings": 2048,
}


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_size_64_with_prompts_of_several_hundred_tokens(tmp_path, dtype):
    """Head size 64, three query heads per key/value head, prompts of 150 to 700 tokens in one step (in
    bfloat16: the tcgen05 attention with two query tiles per CTA, over page borders and ragged ends), then
    tokens one by one for all, and a second prompt chunk on top of a first."""
    from dryft_flash_infer_b200 import Engine, StepEntry

    cfg = TINY_D
    weights = plain_model.random_weights(cfg, seed=12, matrix_std=0.05, norm_std=0.1)
    folder = write_model(tmp_path, cfg, weights)
    ref_w = reference_weights(weights, dtype)
    engine = Engine(folder, dtype=dtype, max_tokens=4096)
    prompts = prompts_for(cfg, [700, 150, 257, 385], seed=5)
    want = [plain_model.forward(cfg, ref_w, p) for p in prompts]
    slots = [engine.open_slot() for _ in prompts]
    places = [[0, len(p) // 2, len(p) - 5] for p in prompts]
    logits = engine.step([StepEntry(s, p[:-4], w) for s, p, w in zip(slots, prompts, places)])
    at = 0
    for i, w in enumerate(places):
        for place in w:
            assert_close(logits[at], want[i][place], dtype, f"prompt {i} place {place}")
            at += 1
    for t in (4, 3):
        logits = engine.step([StepEntry(s, [p[len(p) - t]], [0]) for s, p in zip(slots, prompts)])
        for i, p in enumerate(prompts):
            assert_close(logits[i], want[i][len(p) - t], dtype, f"decode {i} -{t}")
    for s in slots:
        engine.close_slot(s)
    # a prompt in two shares: the second attends over the first's keys through the cache
    slot = engine.open_slot()
    p = prompts[0]
    engine.step([StepEntry(slot, p[:300], [])])
    logits = engine.step([StepEntry(slot, p[300:], [0, len(p) - 301])])
    assert_close(logits[0], want[0][300], dtype, "second share, first place")
    assert_close(logits[1], want[0][len(p) - 1], dtype, "second share, last place")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_short_prompt_steps_replayed_as_graphs(folders, name, dtype):
    """Prompt steps of unequal sizes that share one padded shape: the first runs kernel by kernel, the
    second is captured, the others are replays of that graph on the same buffers.  Every one of them
    must give the logits of the plain implementation, whatever the step before left in the buffers;
    one sequence stays live throughout, so a stray write of a spare row into its pages would show in
    its later share; and with graphs switched off the engine must agree too."""
    from dryft_flash_infer_b200 import StepEntry

    folder, cfg, weights = folders[name]
    ref_w = reference_weights(weights, dtype)
    engine = make_engine(folder, dtype, max_tokens=64 * 24, cuda_graph=True)
    assert engine.stepper.graphs is not None
    plain_engine = make_engine(folder, dtype, max_tokens=64 * 24, cuda_graph=False)
    assert plain_engine.stepper.graphs is None
    long_prompt = prompts_for(cfg, [130], seed=77)[0]
    want_long = plain_model.forward(cfg, ref_w, long_prompt)
    keeper = engine.open_slot()
    fed = 0
    # every round: 3 fresh prompts and a share of the long one, 4 sequences and 4 wanted places in 128 rows
    for round_, (lengths, share) in enumerate([((5, 40, 31), 20), ((20, 30, 33), 9), ((1, 2, 60), 50), ((64, 3, 7), 51)]):
        prompts = prompts_for(cfg, lengths, seed=200 + round_)
        slots = [engine.open_slot() for _ in prompts]
        entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        entries.insert(1, StepEntry(keeper, long_prompt[fed:fed + share], [share - 1]))
        logits = engine.step(entries)
        assert logits.shape[0] == 4
        rows = [0, 2, 3]
        for row, p in zip(rows, prompts):
            assert_close(logits[row], plain_model.forward(cfg, ref_w, p)[len(p) - 1], dtype, f"round {round_}, {len(p)} tokens")
        assert_close(logits[1], want_long[fed + share - 1], dtype, f"round {round_}, the long prompt's share")
        fed += share
        other_slots = [plain_engine.open_slot() for _ in prompts]
        other = plain_engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(other_slots, prompts)])
        assert_close(logits[rows], other, dtype, f"round {round_}, against the engine without graphs")
        for s in slots:
            engine.close_slot(s)
        for s in other_slots:
            plain_engine.close_slot(s)
    assert fed == 130
    assert engine.stepper.graphs.replays == 3 and len(engine.stepper.graphs.shapes) == 1
    engine.close_slot(keeper)
    engine.cache.book.check()
    assert engine.cache.live_slots == 0


def test_prompts_with_every_product_on_our_own_kernels(tmp_path, monkeypatch):
    """``DRYFT_PREFILL_GEMM=own``: a prompt's qkv, o, gate_up and down products all run on the pair kernel
    (the library's product is the default only because it is faster on these shapes).  Same logits."""
    from dryft_flash_infer_b200 import StepEntry
    from dryft_flash_infer_b200.ops import kernels

    weights = plain_model.random_weights(TINY_D, seed=5, matrix_std=0.05, norm_std=0.1)
    folder = write_model(tmp_path, TINY_D, weights)
    ref_w = reference_weights(weights, "bfloat16")
    prompts = prompts_for(TINY_D, [300, 70, 129], seed=3)
    monkeypatch.setattr(kernels, "PREFILL_GEMM", "own")
    calls = []
    real = kernels.pair_linear
    monkeypatch.setattr(kernels, "pair_linear", lambda x, w, swiglu=False: (calls.append(swiglu), real(x, w, swiglu))[1])
    engine = make_engine(folder, "bfloat16", max_tokens=64 * 12, cuda_graph=False)
    slots = [engine.open_slot() for _ in prompts]
    logits = engine.step([StepEntry(s, p, [0, len(p) - 1]) for s, p in zip(slots, prompts)])
    layers = TINY_D["num_hidden_layers"]
    assert calls.count(True) == layers and calls.count(False) == 3 * layers        # gate_up; qkv, o, down
    assert kernels.pair_error() == 0
    for i, p in enumerate(prompts):
        want = plain_model.forward(TINY_D, ref_w, p)
        assert_close(logits[2 * i], want[0], "bfloat16", f"prompt {i}, first place")
        assert_close(logits[2 * i + 1], want[len(p) - 1], "bfloat16", f"prompt {i}, last place")


def test_graphs_of_several_shapes_take_turns_and_the_oldest_goes(folders, monkeypatch):
    """Shapes used in turn share one memory pool for their graphs, and only a few are kept: a shape that was
    dropped starts again from its first use.  Every step still gives the plain implementation's logits."""
    from dryft_flash_infer_b200 import StepEntry
    from dryft_flash_infer_b200.engine import prefill

    folder, cfg, weights = folders["B"]
    ref_w = reference_weights(weights, "bfloat16")
    monkeypatch.setattr(prefill, "MAX_GRAPHS", 2)
    engine = make_engine(folder, "bfloat16", max_tokens=64 * 16, cuda_graph=True)
    graphs = engine.stepper.graphs
    turns = [(70,), (140,), (70,), (140,), (70, 3), (140,), (70,), (70,), (70, 5), (70, 3)]
    for turn, lengths in enumerate(turns):
        prompts = prompts_for(cfg, lengths, seed=400 + turn)
        slots = [engine.open_slot() for _ in prompts]
        logits = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        for row, p in enumerate(prompts):
            assert_close(logits[row], plain_model.forward(cfg, ref_w, p)[len(p) - 1], "bfloat16", f"turn {turn}, {len(p)} tokens")
        for s in slots:
            engine.close_slot(s)
        assert len(graphs.shapes) <= 2
    # with room for two shapes, the one whose last use is the longest ago goes: (128, 2, 1) at turn 4,
    # (128, 4, 2) at turn 6, (256, 2, 1) at turn 8; a shape that comes back starts from its first use.
    # Replays (every use of a shape after its first since it came): turns 2, 3, 5, 7 and 9.
    assert graphs.replays == 5
    engine.cache.book.check()


def _teacher_forced_gap(cfg, ref_w, prompt, tokens) -> float:
    """How far below the plain implementation's best logit the chosen tokens lie at most, each judged on
    the sequence of the tokens chosen before it."""
    seq, worst = list(prompt), 0.0
    for token in tokens:
        logits = plain_model.forward(cfg, ref_w, seq)[-1]
        worst = max(worst, float(logits.max() - logits[token]))
        seq.append(token)
    return worst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_generation_with_a_live_set_that_shrinks_and_slots_used_again(folders, name, dtype):
    """The path generation really takes: fixed decode buffers and CUDA graphs, with requests of unequal
    prompts and unequal lengths of output, three at a time.  Sequences end at different steps, so the
    batch size of the decode buffers changes in mid-batch and the tokens are fed from the host again;
    the next batch takes the slots and pages of the one before, which are full of NaN or of old keys."""
    from dryft_flash_infer_b200 import Request

    folder, cfg, weights = folders[name]
    ref_w = reference_weights(weights, dtype)
    engine = make_engine(folder, dtype, max_tokens=64 * 12, cuda_graph=True)
    assert engine.decoder.use_graph
    lengths = [5, 70, 9, 17, 1, 64, 33, 2]
    news = [3, 12, 5, 8, 1, 7, 12, 4]
    prompts = prompts_for(cfg, lengths, seed=61)
    requests = [Request(p, n, request_id=i) for i, (p, n) in enumerate(zip(prompts, news))]
    engine.generate_requests(requests, max_batch=3)
    assert engine.cache.live_slots == 0
    engine.cache.book.check()
    sizes = {b.n for b in engine.decoder.batches.values()}
    assert {1, 2, 3} <= sizes                                   # the live set did shrink
    for r, n in zip(requests, news):
        assert len(r.output) == n and r.finish_reason == "length"
        if dtype == "float32":
            assert r.output == plain_model.greedy_continue(cfg, ref_w, r.prompt, n), f"request {r.request_id}"
        else:
            assert _teacher_forced_gap(cfg, ref_w, r.prompt, r.output) <= BF16_TIE_GAP, f"request {r.request_id}"
    # the same with stop tokens taken from the plain implementation's own continuation, so that the
    # place where each sequence must stop is known
    plain = [plain_model.greedy_continue(cfg, ref_w, p, n) for p, n in zip(prompts, news)]
    again = [Request(p, n, stop_token_ids=(out[min(2, n - 1)],), request_id=i)
             for i, (p, n, out) in enumerate(zip(prompts, news, plain))]
    engine.generate_requests(again, max_batch=3)
    assert engine.cache.live_slots == 0
    for r, out in zip(again, plain):
        stop = r.stop_token_ids[0]
        if dtype == "float32":
            cut = out.index(stop) + 1
            assert r.output == out[:cut] and r.finish_reason == "stop"
        else:
            assert _teacher_forced_gap(cfg, ref_w, r.prompt, r.output) <= BF16_TIE_GAP
            assert stop not in r.output[:-1]
            assert r.finish_reason == ("stop" if r.output[-1] == stop else "length")


def test_a_wait_that_runs_out_reaches_the_host_as_an_exception(folders):
    """Each tcgen05 library has a one-CTA kernel that waits (a try or two) on a barrier nothing arrives on,
    records its code as a real kernel's wait would, frees its tensor memory and returns.  The code must
    come back with the next results the host reads, as an exception, and be cleared by that."""
    from dryft_flash_infer_b200 import StepEntry
    from dryft_flash_infer_b200.ops import kernels
    from dryft_flash_infer_b200.sampling import SamplingParams

    folder, cfg, weights = folders["B"]
    engine = make_engine(folder, "bfloat16", max_tokens=512, cuda_graph=True)
    engine.check_status()
    for unit, head_dim, code in (("gemm_decode", 128, 41), ("gemm_pair", 128, 42), ("attention_prefill_tc", 64, 43),
                                 ("attention_decode", 32, 45)):
        kernels.wait_selftest(unit, limit=2, code=code, head_dim=head_dim)
        with pytest.raises(kernels.KernelError, match=f"{unit} .wait code {code}."):
            engine.check_status()
        engine.check_status()                                   # read once, cleared
    assert kernels.tc_error(reset=False) == 0 and kernels.pair_error(reset=False) == 0
    assert kernels.attention_tc_error(64, reset=False) == 0
    # through generation's decode step: the code travels with the step's tokens
    prompt = prompts_for(cfg, [9], seed=4)[0]
    slot = engine.open_slot()
    logits = engine.step([StepEntry(slot, prompt, [len(prompt) - 1])])
    first = engine.select(logits, [0], 0, SamplingParams())
    handle = engine.decode_launch([slot], first, [0], 1, SamplingParams())
    kernels.wait_selftest("gemm_decode", limit=1, code=44)
    second = engine.decode_launch([slot], None, [0], 2, SamplingParams())
    handle.result()                                             # launched before the failure: clean
    with pytest.raises(kernels.KernelError, match="wait code 44"):
        second.result()
    engine.close_slot(slot)
    # and the engine goes on: the same request again gives the plain implementation's tokens
    got = [r[0] for r in engine.generate([prompt], 4)]
    assert _teacher_forced_gap(cfg, bf16_weights(weights), prompt, got) <= BF16_TIE_GAP
    # a word set by the host shows the same way
    kernels.status_words()[6] = 9
    with pytest.raises(kernels.KernelError, match="word 6"):
        engine.check_status()


def test_sharded_model_folders_load_through_the_engine(tmp_path):
    """A model in two shards with ``model.safetensors.index.json`` gives the logits of the same model in
    one file; a tensor that two shards hold, and a shard the index names but the folder lacks, are errors."""
    import json
    import shutil

    from dryft_flash_infer_b200 import Engine, Qwen3Config, StepEntry
    from dryft_flash_infer_b200.weights import SafetensorsError, write_safetensors

    cfg = plain_model.TINY_A
    weights = plain_model.random_weights(cfg, seed=14, matrix_std=0.06, norm_std=0.1)
    names = sorted(weights)
    parts = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
             "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    folder = tmp_path / "sharded"
    Qwen3Config.from_dict(cfg).save(folder)
    for file, held in parts.items():
        write_safetensors(folder / file, ((n, weights[n]) for n in held))
    index = {"metadata": {}, "weight_map": {n: file for file, held in parts.items() for n in held}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    prompt = prompts_for(cfg, [21], seed=2)[0]
    engine = Engine(folder, dtype="float32", max_tokens=128)
    slot = engine.open_slot()
    logits = engine.step([StepEntry(slot, prompt, list(range(len(prompt))))])
    assert_close(logits, plain_model.forward(cfg, weights, prompt), "float32", "sharded model")
    # the same tensor in both shards
    twice = tmp_path / "twice"
    shutil.copytree(folder, twice)
    write_safetensors(twice / "model-00002-of-00002.safetensors",
                      ((n, weights[n]) for n in parts["model-00002-of-00002.safetensors"] + [names[0]]))
    with pytest.raises(SafetensorsError, match=names[0].replace(".", r"\.")):
        Engine(twice, dtype="float32", max_tokens=128)
    # a shard that is not there
    lost = tmp_path / "lost"
    shutil.copytree(folder, lost)
    (lost / "model-00001-of-00002.safetensors").unlink()
    with pytest.raises((SafetensorsError, FileNotFoundError), match="model-00001-of-00002"):
        Engine(lost, dtype="float32", max_tokens=128)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_steps_of_a_few_rows_keep_the_decode_products(folders, dtype):
    """Prompt steps of up to 64 rows are padded to 16, 32 or 64 rows, so that their products run the decode
    kernels; each shape is captured at its second use and replayed afterwards.  Same logits as the plain
    implementation at every use, with a sequence that stays live across the steps."""
    from dryft_flash_infer_b200 import StepEntry

    folder, cfg, weights = folders["B"]
    ref_w = reference_weights(weights, dtype)
    engine = make_engine(folder, dtype, max_tokens=64 * 16, cuda_graph=True)
    long_prompt = prompts_for(cfg, [90], seed=5)[0]
    want_long = plain_model.forward(cfg, ref_w, long_prompt)
    keeper, fed = engine.open_slot(), 0
    for round_, (lengths, share) in enumerate([((3, 5), 4), ((2, 9), 3), ((20,), 7), ((1, 6), 2), ((11, 12), 30),
                                               ((4, 4), 5), ((17,), 10), ((30, 20), 11)]):
        prompts = prompts_for(cfg, lengths, seed=300 + round_)
        slots = [engine.open_slot() for _ in prompts]
        entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        entries.append(StepEntry(keeper, long_prompt[fed:fed + share], [0, share - 1]))
        logits = engine.step(entries)
        for row, p in enumerate(prompts):
            assert_close(logits[row], plain_model.forward(cfg, ref_w, p)[len(p) - 1], dtype, f"round {round_}, {len(p)} tokens")
        assert_close(logits[len(prompts)], want_long[fed], dtype, f"round {round_}, the long prompt's share, first place")
        assert_close(logits[len(prompts) + 1], want_long[fed + share - 1], dtype, f"round {round_}, the share's last place")
        fed += share
        for s in slots:
            engine.close_slot(s)
    shapes = sorted(engine.stepper.graphs.shapes)
    assert [shape[0] for shape in shapes] == [16, 32, 64] and engine.stepper.graphs.replays >= 3
    engine.close_slot(keeper)
    engine.cache.book.check()


def test_the_words_about_the_next_product_change_no_logit(wide_model, monkeypatch):
    """Decode kernels are told which weights the step streams after them (the feed-forward's after the
    mixer's, the next layer's after that, the output head's at the end) and ask some of them into L2.
    With the hints off the step's logits are the same bit for bit, launch by launch and through the graph."""
    from dryft_flash_infer_b200 import StepEntry
    from dryft_flash_infer_b200.ops import kernels

    folder, prompts, _, _ = wide_model            # widths at which the products have tiles beyond their first ring
    prompts = [p[:70] for p in prompts[:3]]
    seen = {}
    for tiles in (4, 0):
        monkeypatch.setattr(kernels, "NEXT_TILES", tiles)
        given = []
        real = kernels.NextWeights.hint
        monkeypatch.setattr(kernels.NextWeights, "hint", lambda self, rows: given.append(real(self, rows)) or given[-1])
        for graph in (False, True):
            engine = make_engine(folder, "bfloat16", max_tokens=64 * 8, cuda_graph=graph)
            assert engine.decoder.use_graph == graph
            slots = [engine.open_slot() for _ in prompts]
            rows = [engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])]
            for t in range(3):
                rows.append(engine.step([StepEntry(s, [7 + t + i], [0]) for i, s in enumerate(slots)]))
            seen[tiles, graph] = torch.cat([r.float().cpu() for r in rows])
        monkeypatch.setattr(kernels.NextWeights, "hint", real)
        # hints were given (and were real ones) exactly when they are on
        assert any(h is not None for h in given) == (tiles > 0)
    assert torch.equal(seen[4, False], seen[0, False])
    assert torch.equal(seen[4, True], seen[0, True])


TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 72, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 80, "intermediate_size": 100, "vocab_size": 257, "rope_theta": 700.0,
    "rms_norm_eps": 2e-5, "tie_word_embeddings": True, "hidden_act": "silu", "max_position_embeddings": 2048,
}


@pytest.mark.parametrize("graph", [True, False])
@pytest.mark.parametrize("hidden, inter", [(72, 100), (100, 56), (100, 100)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_widths_that_are_no_multiples_of_eight(tmp_path, dtype, hidden, inter, graph):
    """An intermediate size or a width of 100: the TMA-fed products take inner sizes in steps of 8 only, so
    these products run on the plain kernel, and a product before a norm must not be asked to fuse with it
    when its own inner size is not one of those (the down projection after a width that is)."""
    from dryft_flash_infer_b200 import Engine, StepEntry

    cfg = dict(TINY_E, hidden_size=hidden, intermediate_size=inter)
    weights = plain_model.random_weights(cfg, seed=hidden + inter, matrix_std=0.06, norm_std=0.1)
    folder = write_model(tmp_path, cfg, weights)
    ref_w = reference_weights(weights, dtype)
    engine = Engine(folder, dtype=dtype, max_tokens=64 * 12, cuda_graph=graph)
    prompts = prompts_for(cfg, [65, 3, 63, 17], seed=5)
    want = [plain_model.forward(cfg, ref_w, p) for p in prompts]
    slots = [engine.open_slot() for _ in prompts]
    logits = engine.step([StepEntry(s, p[:-2], [len(p) - 3]) for s, p in zip(slots, prompts)])
    for i, p in enumerate(prompts):
        assert_close(logits[i], want[i][len(p) - 3], dtype, f"prefill {i}")
    for t in (2, 1):
        logits = engine.step([StepEntry(s, [p[len(p) - t]], [0]) for s, p in zip(slots, prompts)])
        for i, p in enumerate(prompts):
            assert_close(logits[i], want[i][len(p) - t], dtype, f"decode {i} -{t}")
    engine.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_live_set_of_more_than_eight_runs_on_buffers_with_places_to_spare(folders, name, dtype):
    """Eleven requests at once with unequal lengths of output: decode steps of 11, 10, 9 sequences run on
    buffers of 16 places (``decode_places``), the places past the live sequences filled with sequences
    of one token on the null page.  Every request's tokens are the plain implementation's, the filling's are
    never seen, and a toy check that the sizes of buffers are the few expected ones."""
    from dryft_flash_infer_b200 import Request
    from dryft_flash_infer_b200.engine.decode import decode_places

    assert [decode_places(n) for n in (1, 2, 3, 7, 8, 9, 11, 16, 17, 33, 64, 65, 100)] == \
        [1, 2, 3, 7, 8, 16, 16, 16, 32, 64, 64, 96, 128]
    folder, cfg, weights = folders[name]
    ref_w = reference_weights(weights, dtype)
    engine = make_engine(folder, dtype, max_tokens=64 * 2 * 11, max_seqs=11, cuda_graph=True)
    lengths = [5, 70, 9, 17, 1, 64, 33, 2, 40, 3, 65]
    news = [3, 14, 5, 8, 2, 7, 14, 4, 9, 11, 6]
    prompts = prompts_for(cfg, lengths, seed=77)
    requests = [Request(p, n, request_id=i) for i, (p, n) in enumerate(zip(prompts, news))]
    engine.generate_requests(requests, max_batch=11)
    assert engine.cache.live_slots == 0
    engine.cache.book.check()
    sizes = sorted({b.n for b in engine.decoder.batches.values()})
    assert set(sizes) <= {1, 2, 3, 4, 5, 6, 7, 8, 16} and {8, 16} <= set(sizes), sizes
    for r, n in zip(requests, news):
        assert len(r.output) == n
        if dtype == "float32":
            assert r.output == plain_model.greedy_continue(cfg, ref_w, r.prompt, n), f"request {r.request_id}"
        else:
            assert _teacher_forced_gap(cfg, ref_w, r.prompt, r.output) <= BF16_TIE_GAP, f"request {r.request_id}"
    # the step function on the same buffers: nine single-token steps' logits against the plain implementation
    from dryft_flash_infer_b200 import StepEntry
    nine = prompts_for(cfg, [12, 3, 30, 8, 64, 65, 2, 19, 7], seed=78)
    slots = [engine.open_slot() for _ in nine]
    engine.step([StepEntry(s, p[:-1], []) for s, p in zip(slots, nine)])
    rows = engine.step([StepEntry(s, [p[-1]], [0]) for s, p in zip(slots, nine)])
    assert rows.shape[0] == 9
    for i, p in enumerate(nine):
        assert_close(rows[i], plain_model.forward(cfg, ref_w, p)[-1], dtype, f"nine at once, sequence {i}")


TINY_F = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 96, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 136, "vocab_size": 157, "rope_theta": 30000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "hidden_act": "silu", "max_position_embeddings": 4096,
}


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_a_length_at_which_the_attention_launch_changes(tmp_path, dtype):
    """One sequence decoded from 2,040 to 2,056 keys on the fixed buffers: at 2,048 the step says another
    limit, the attention kernel is launched in another shape (clusters of sixteen CTAs in bfloat16) and a
    second graph is captured on the same buffers.  Every token's logits against the plain implementation;
    then a second, short sequence goes back to the first limit's graph."""
    from dryft_flash_infer_b200 import Engine, StepEntry
    from dryft_flash_infer_b200.ops import kernels

    cfg = TINY_F
    weights = plain_model.random_weights(cfg, seed=21, matrix_std=0.05, norm_std=0.1)
    folder = write_model(tmp_path, cfg, weights)
    ref_w = reference_weights(weights, dtype)
    engine = Engine(folder, dtype=dtype, max_tokens=4096, max_context=4096)
    prompt = prompts_for(cfg, [2056], seed=8)[0]
    short = prompts_for(cfg, [70], seed=9)[0]
    want = plain_model.forward(cfg, ref_w, prompt, places=list(range(2039, 2056)))
    want_short = plain_model.forward(cfg, ref_w, short, places=[68, 69])
    slot = engine.open_slot()
    logits = engine.step([StepEntry(slot, prompt[:2040], [2039])])
    assert_close(logits[0], want[0], dtype, "the prompt's last place")
    for i in range(2040, 2056):
        logits = engine.step([StepEntry(slot, [prompt[i]], [0])])
        assert_close(logits[0], want[i - 2039], dtype, f"token {i}")
    for batch in engine.decoder.batches.values():          # (none when graphs are switched off)
        if batch.use_graph:
            assert sorted(batch.graphs) == [kernels.DECODE_KV_STEPS[0], 4096]
            assert all(graph is not False for graph, _ in batch.graphs.values())
    engine.close_slot(slot)
    slot = engine.open_slot()
    engine.step([StepEntry(slot, short[:68], [])])
    for i in (68, 69):
        logits = engine.step([StepEntry(slot, [short[i]], [0])])
        assert_close(logits[0], want_short[i - 68], dtype, f"short sequence, token {i}")
    engine.close_slot(slot)
    engine.check_status()
