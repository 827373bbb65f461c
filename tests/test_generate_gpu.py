"""Generation through the Python entry point and the engine: greedy tokens equal the plain
implementation's; sampling does not depend on the batch; the CUDA-graph decode path equals
the eager one; a pool too small for everyone preempts and still gives the same tokens."""
import pytest
import torch

import harness
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu


def model_dir(tmp_path, name):
    cfg, w = harness.weights_for(name)
    return tiny_configs.write_model_dir(tmp_path / name, cfg, {k: v.to(torch.bfloat16) for k, v in w.items()})


def prompts_for(name):
    cfg = tiny_configs.ALL[name][0]
    lengths = (5, 17, 33) if name == "A" else (1, 9, 24, 40)
    return [tiny_configs.make_ids(cfg, n, seed=50 + i) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    from torchlet_b200 import LLM

    folder = model_dir(tmp_path, name)
    page = tiny_configs.ALL[name][1]["page_size"]
    llm = LLM(folder, max_decode_slots=4, kv_block_size=page, dtype=dtype, max_seq_len=128)
    prompts = prompts_for(name)
    new = 8 if name == "A" else 12
    outputs = llm.generate(prompts, max_new_tokens=new)
    assert llm.engine.runner.graph_steps > 0  # decode went through the captured graph
    cfg, w = harness.weights_for(name)
    for prompt, got in zip(prompts, outputs):
        assert len(got) == new
        if dtype == "float32":
            assert got == plain_model.greedy_generate(cfg, w, prompt, new)
        else:
            # bfloat16 may flip a near-tie: every token must be within rounding of the best
            ids = list(prompt)
            for token in got:
                logits = plain_model.forward_logits(cfg, w, ids)[-1]
                assert logits[token] >= logits.max() - 2.5e-2 * logits.abs().max()
                ids.append(token)
    llm.engine.runner.cache.check()
    assert llm.engine.runner.cache.live_requests() == []


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_decode_equals_eager_decode(tmp_path, dtype):
    from torchlet_b200 import LLM, SamplingParams

    folder = model_dir(tmp_path, "B")
    prompts = prompts_for("B")
    params = [SamplingParams(max_new_tokens=20, temperature=t, seed=11 + i) for i, t in enumerate((0.0, 0.8, 0.0, 1.1))]
    outs = []
    for graph in (True, False):
        llm = LLM(folder, max_decode_slots=4, kv_block_size=8, dtype=dtype, max_seq_len=128, cuda_graph=graph)
        outs.append(llm.generate(prompts, sampling_params=params))
        assert (llm.engine.runner.graph_steps > 0) == graph
    if dtype == "float32":
        assert outs[0] == outs[1]
    else:
        same = sum(a == b for x, y in zip(*outs) for a, b in zip(x, y))
        assert same >= 0.8 * sum(len(x) for x in outs[0])


def test_coroutines_that_arrive_one_after_the_other(tmp_path):
    """``await llm.agenerate(...)`` from three coroutines that start at different times, the
    reference's own demonstration (v10_triton_paged_gqa/llm.py:113-140): one engine loop serves
    them together, and in float32 every output equals the synchronous ``generate`` of the same
    prompt alone; ``shutdown`` ends the loop with nothing held."""
    import asyncio

    from torchlet_b200 import LLM, SamplingParams

    folder = model_dir(tmp_path, "B")
    prompts = prompts_for("B")
    params = [SamplingParams(max_new_tokens=14 + 3 * i, temperature=t, seed=21 + i)
              for i, t in enumerate((0.0, 0.8, 0.0, 1.1))]
    llm = LLM(folder, max_decode_slots=3, kv_block_size=8, dtype="float32", max_seq_len=128)
    alone = [llm.generate([p], sampling_params=[sp])[0] for p, sp in zip(prompts, params)]

    async def main():
        try:
            tasks = []
            for prompt, sp in zip(prompts, params):
                tasks.append(asyncio.create_task(llm.agenerate([prompt], sampling_params=[sp])))
                await asyncio.sleep(0.002)
            return await asyncio.gather(*tasks)
        finally:
            await llm.shutdown()

    before = llm.engine.scheduler.stats.steps
    together = asyncio.run(main())
    assert [out[0] for out in together] == alone
    stats = llm.engine.scheduler.stats
    assert stats.steps - before < sum(sp.max_new_tokens for sp in params), "the coroutines' requests never shared a step"
    assert stats.peak_running == 3  # four callers, three slots: one waited its turn
    llm.engine.runner.cache.check()
    assert llm.engine.runner.cache.live_requests() == [] and llm.engine._task is None


def _write_tokenizer(folder, vocab_size):
    """A word-level tokenizer with the special tokens and a chat template of the kind the
    reference's model has, written locally (tokenizer.json + tokenizer_config.json)."""
    import json

    from tokenizers import Tokenizer, models, pre_tokenizers

    words = ["<unk>", "<|im_start|>", "<|im_end|>", "user", "assistant", "hello", "world", "what", "is", "the",
             "nearest", "star"]
    words += [f"w{i}" for i in range(vocab_size - len(words))]
    tokenizer = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tokenizer.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tokenizer.save(str(folder / "tokenizer.json"))
    template = ("{% for m in messages %}<|im_start|> {{ m['role'] }} {{ m['content'] }} <|im_end|> {% endfor %}"
                "{% if add_generation_prompt %}<|im_start|> assistant {% endif %}")
    (folder / "tokenizer_config.json").write_text(json.dumps({
        "tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<|im_end|>", "unk_token": "<unk>",
        "chat_template": template}))
    return words


def test_text_prompts_through_the_tokenizer(tmp_path):
    """Text in, text out, as the reference's entry point (v10_triton_paged_gqa/llm.py:84-110): the
    folder's tokenizer, its chat template around a single user turn, the stop ids from the
    tokenizer (eos and <|im_end|>), the output decoded without special tokens; equal to the same
    ids given as ids, also from a coroutine."""
    import asyncio

    from torchlet_b200 import LLM

    folder = model_dir(tmp_path, "A")
    words = _write_tokenizer(folder, tiny_configs.ALL["A"][0]["vocab_size"])
    llm = LLM(folder, max_decode_slots=4, kv_block_size=16, dtype="float32", max_seq_len=128)
    assert llm.tokenizer is not None and llm.stop_ids == {2}
    prompts = ["hello world", "what is the nearest star"]
    ids = llm._encode(prompts)
    assert ids[0] == [1, 3, 5, 6, 2, 1, 4] and ids[1][:3] == [1, 3, 7] and ids[1][-2:] == [1, 4]
    texts = llm.generate(prompts, max_new_tokens=12)
    tokens = llm.generate(ids, max_new_tokens=12)  # the same ids as ids: the tokenizer's stop ids apply as well
    assert all(isinstance(t, str) for t in texts) and len(texts) == 2
    for text, produced in zip(texts, tokens):
        assert 2 not in produced and len(produced) <= 12  # a stop token ends the request and is not emitted
        assert text == " ".join(words[t] for t in produced if t > 2)
    assert asyncio.run(_one_coroutine(llm, prompts)) == texts
    cfg, w = harness.weights_for("A")
    plain = plain_model.greedy_generate(cfg, w, ids[0], 12)
    cut = plain.index(2) if 2 in plain else len(plain)
    assert tokens[0] == plain[:cut]


async def _one_coroutine(llm, prompts):
    try:
        return await llm.agenerate(prompts, max_new_tokens=12)
    finally:
        await llm.shutdown()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_shutdown_while_requests_decode(tmp_path, dtype):
    """``shutdown`` in the middle of decoding, a step launched ahead still in flight: the waiting
    coroutine gets ``CancelledError``, every page and slot is back, and the same engine then
    generates what a fresh one generates."""
    import asyncio

    from torchlet_b200 import LLM

    folder = model_dir(tmp_path, "B")
    prompts = prompts_for("B")
    llm = LLM(folder, max_decode_slots=4, kv_block_size=8, dtype=dtype, max_seq_len=512)
    fresh = llm.generate(prompts, max_new_tokens=10)

    async def main():
        task = asyncio.create_task(llm.agenerate(prompts, max_new_tokens=400, sampling_params=None))
        while llm.engine.scheduler.stats.decode_tokens < 40:  # well into decoding, far from done
            await asyncio.sleep(0)
        assert llm.engine.steps_ahead > 0 and not task.done()
        await llm.shutdown()
        with pytest.raises(asyncio.CancelledError):
            await task

    before = llm.engine.scheduler.stats.decode_tokens
    asyncio.run(main())
    assert 40 <= llm.engine.scheduler.stats.decode_tokens - before + 40 < 4 * 400
    torch.cuda.synchronize()
    llm.engine.runner.cache.check()
    assert llm.engine.runner.cache.live_requests() == [] and not llm.engine.scheduler.has_work()
    assert llm.engine.runner.cache.num_free_slots == 4
    assert llm.generate(prompts, max_new_tokens=10) == fresh


def test_sampling_does_not_depend_on_the_batch(tmp_path):
    from torchlet_b200 import LLM, SamplingParams

    folder = model_dir(tmp_path, "B")
    prompts = prompts_for("B")
    params = [SamplingParams(max_new_tokens=12, temperature=0.8, seed=100 + i) for i in range(len(prompts))]
    llm = LLM(folder, max_decode_slots=4, kv_block_size=8, dtype="float32", max_seq_len=128)
    together = llm.generate(prompts, sampling_params=params)
    alone = [llm.generate([p], sampling_params=[sp])[0] for p, sp in zip(prompts, params)]
    assert together == alone
    other_seed = llm.generate([prompts[3]], sampling_params=[SamplingParams(max_new_tokens=12, temperature=0.8, seed=5)])[0]
    assert other_seed != alone[3]
    # the first draw follows the plain rule
    cfg, w = harness.weights_for("B")
    logits = plain_model.forward_logits(cfg, w, prompts[2])[-1]
    scores = plain_model.temperature_scores(logits, 0.8, 102, 0)
    assert scores[alone[2][0]] >= max(scores) - 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_one_step_ahead_equals_stepping(tmp_path, dtype):
    """``Engine.run`` launches a decode step before it has read the tokens of the one before;
    it must give what synchronous ``step()`` calls give, also when requests end by a stop
    token (one lane of the step under way is void then), by their token limit, and when new
    requests join as slots come free."""
    from torchlet_b200 import LLM, SamplingParams
    from torchlet_b200.engine.scheduler import Request

    folder = model_dir(tmp_path, "B")
    cfg = tiny_configs.ALL["B"][0]
    prompts = [tiny_configs.make_ids(cfg, n, seed=80 + i) for i, n in enumerate((3, 21, 9, 30, 14, 6))]

    def requests(stops):
        limits = (25, 9, 31, 16, 12, 40)
        return [Request(list(p), SamplingParams(max_new_tokens=m, temperature=t, seed=7 + i, stop_token_ids=stops))
                for i, (p, m, t) in enumerate(zip(prompts, limits, (0.0, 0.9, 0.0, 0.7, 0.0, 1.2)))]

    def stepping(stops):
        llm = LLM(folder, max_decode_slots=3, kv_block_size=8, dtype=dtype, max_seq_len=128)
        reqs = requests(stops)
        llm.engine.add_requests(reqs)
        while llm.engine.scheduler.has_work():
            llm.engine.step()
        llm.engine.runner.cache.check()
        return [r.output_tokens for r in reqs]

    def running(stops):
        llm = LLM(folder, max_decode_slots=3, kv_block_size=8, dtype=dtype, max_seq_len=128)
        reqs = requests(stops)
        llm.engine.generate(reqs)
        llm.engine.runner.cache.check()
        assert llm.engine.runner.cache.live_requests() == []
        assert llm.engine.runner.graph_steps > 0 and llm.engine.steps_ahead > 0
        return [r.output_tokens for r in reqs]

    free = stepping(())
    assert [len(x) for x in free] == [25, 9, 31, 16, 12, 40]
    assert running(()) == free
    # tokens that really occur, some of them early, as stop tokens
    stops = tuple({free[0][6], free[2][3], free[5][20], free[3][15]})
    cut = stepping(stops)
    assert any(len(a) < len(b) for a, b in zip(cut, free))
    assert running(stops) == cut


def test_small_pool_preempts_and_gives_the_same_tokens(tmp_path):
    from torchlet_b200 import LLM

    folder = model_dir(tmp_path, "A")
    cfg = tiny_configs.ALL["A"][0]
    prompts = [tiny_configs.make_ids(cfg, n, seed=70 + i) for i, n in enumerate((40, 37, 45, 30, 22))]
    roomy = LLM(folder, max_decode_slots=4, kv_block_size=16, dtype="float32", max_seq_len=128)
    want = roomy.generate(prompts, max_new_tokens=30)
    # 9 usable pages of 16 tokens: not enough for four requests of ~70 tokens
    tight = LLM(folder, max_decode_slots=4, kv_block_size=16, max_num_blocks=10, dtype="float32", max_seq_len=128,
                max_num_batched_tokens=48)
    got = tight.generate(prompts, max_new_tokens=30)
    assert got == want
    assert tight.engine.scheduler.stats.preemptions > 0
    tight.engine.runner.cache.check()
    assert tight.engine.runner.cache.pools[0].num_free == 9


def test_a_request_too_large_for_the_pool_fails_alone(tmp_path):
    from torchlet_b200.engine.scheduler import Request
    from torchlet_b200 import LLM, SamplingParams

    folder = model_dir(tmp_path, "A")
    cfg = tiny_configs.ALL["A"][0]
    llm = LLM(folder, max_decode_slots=2, kv_block_size=16, max_num_blocks=4, dtype="float32", max_seq_len=128)
    small = Request(tiny_configs.make_ids(cfg, 10, 1), SamplingParams(max_new_tokens=4))
    big = Request(tiny_configs.make_ids(cfg, 90, 2), SamplingParams(max_new_tokens=4))
    llm.engine.generate([small, big])
    assert small.error is None and len(small.output_tokens) == 4
    assert big.error is not None and "too small" in str(big.error)
    with pytest.raises(ValueError, match="cache positions"):
        llm.generate([tiny_configs.make_ids(cfg, 120, 3)], max_new_tokens=20)


def test_command_line(tmp_path):
    import subprocess
    import sys

    folder = model_dir(tmp_path, "A")
    cmd = [sys.executable, "-m", "torchlet_b200.llm", "--model", str(folder), "--prompt-ids", "1,2,3", "--prompt-ids",
           "9,8", "--max-new-tokens", "5", "--dtype", "float32", "--max-seq-len", "64"]
    out = subprocess.run(cmd, capture_output=True, text=True, cwd=str(harness.tiny_configs.__file__).rsplit("/tests", 1)[0])
    assert out.returncode == 0, out.stderr
    lines = [line for line in out.stdout.splitlines() if line.startswith("[")]
    assert len(lines) == 2 and all(len(eval(line)) == 5 for line in lines)
    cfg, w = harness.weights_for("A")
    assert eval(lines[0]) == plain_model.greedy_generate(cfg, w, [1, 2, 3], 5)


def test_command_line_writes_random_weights_and_serves_three_arrivals(tmp_path):
    """``--random-weights SEED`` writes model.safetensors into a folder that holds only a config.json
    (and here a tokenizer); without prompts the command line does what the reference's does
    (v10_triton_paged_gqa/llm.py:113-140): its three prompts as three coroutines a tenth of a
    second apart, one engine loop, three printed batches."""
    import json
    import subprocess
    import sys

    folder = tmp_path / "fresh"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(tiny_configs.ALL["A"][0]))
    _write_tokenizer(folder, tiny_configs.ALL["A"][0]["vocab_size"])
    root = str(harness.tiny_configs.__file__).rsplit("/tests", 1)[0]
    cmd = [sys.executable, "-m", "torchlet_b200.llm", "--model", str(folder), "--random-weights", "11", "--max-new-tokens",
           "6", "--ignore-eos", "--max-seq-len", "128"]
    out = subprocess.run(cmd, capture_output=True, text=True, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    assert (folder / "model.safetensors").is_file()
    lines = out.stdout.splitlines()
    assert [line for line in lines if line.startswith("batch ")] == ["batch 1:", "batch 2:", "batch 3:"]
    batches = [eval(line) for line in lines if line.startswith("[")]
    assert len(batches) == 3 and all(len(b) == 1 and isinstance(b[0], str) and len(b[0].split()) <= 6 for b in batches)
    # the same folder again, now with its weights: ids in, ids out
    again = subprocess.run([sys.executable, "-m", "torchlet_b200.llm", "--model", str(folder), "--prompt-ids", "5,6,7",
                            "--max-new-tokens", "4", "--ignore-eos", "--max-seq-len", "128"], capture_output=True,
                           text=True, cwd=root)
    assert again.returncode == 0, again.stderr[-2000:]
    assert len(eval([line for line in again.stdout.splitlines() if line.startswith("[")][0])) == 4


def test_entry_point_edges(tmp_path):
    """No inputs, no new tokens, text without a tokenizer, a request longer than the engine takes,
    per-request sampling options, and ``LLM.from_model`` around a model that is already loaded."""
    import asyncio

    from torchlet_b200 import LLM, SamplingParams

    folder = model_dir(tmp_path, "A")
    llm = LLM(folder, max_decode_slots=2, kv_block_size=16, dtype="float32", max_seq_len=64)
    assert llm.tokenizer is None and llm.generate([]) == [] and asyncio.run(llm.agenerate([])) == []
    assert llm.generate([[1, 2, 3]], max_new_tokens=0) == [[]]
    with pytest.raises(ValueError, match="tokenizer"):
        llm.generate(["hello"])
    with pytest.raises(ValueError, match="max_seq_len"):
        llm.generate([[1] * 60], max_new_tokens=10)
    assert llm.engine.runner.cache.live_requests() == [] and not llm.engine.scheduler.has_work()
    # a prompt that fills the engine's length to the last position still gets its one token (which needs no
    # cache position of its own), and equals the plain implementation's
    cfg, w = harness.weights_for("A")
    full = tiny_configs.make_ids(cfg, 64, seed=77)
    assert llm.generate([full], max_new_tokens=1) == [plain_model.greedy_generate(cfg, w, full, 1)]
    with pytest.raises(ValueError, match="max_seq_len"):
        llm.generate([full], max_new_tokens=2)
    params = [SamplingParams(max_new_tokens=3), SamplingParams(max_new_tokens=7, temperature=0.5, seed=3)]
    outs = llm.generate([[5, 6], [7, 8, 9]], sampling_params=params)
    assert [len(o) for o in outs] == [3, 7]
    wrapped = LLM.from_model(llm.model, max_decode_slots=2, kv_block_size=16, max_seq_len=64)
    assert wrapped.engine_config.dtype == "float32" and wrapped.tokenizer is None
    assert wrapped.generate([[5, 6], [7, 8, 9]], sampling_params=params) == outs


def test_a_pool_larger_than_the_memory_is_refused_in_words(tmp_path):
    from torchlet_b200 import LLM
    from torchlet_b200.cache.manager import CacheError

    folder = model_dir(tmp_path, "A")
    with pytest.raises(CacheError, match="GiB are free"):
        LLM(folder, max_decode_slots=4, kv_block_size=16, max_num_blocks=200_000_000, dtype="float32", max_seq_len=128)
