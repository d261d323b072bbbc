"""Generation through the Python entry point and the scheduler, against the plain implementation."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, random_tokens
from plain_minicpm import plain_forward, plain_sample

pytestmark = pytest.mark.gpu


def plain_generate(cfg, w, prompt, steps, temperature=0.0, topk=0, topp=1.0, seed=0, margin=0.0):
    """Continuation by the plain implementation, recomputing the whole sequence for each token.
    Returns (tokens, first step at which the choice was closer than ``margin``, or None)."""
    from infinicore_infer_b200.sampling import uniform_for
    seq, out, doubtful = list(prompt), [], None
    for i in range(steps):
        logits = plain_forward(cfg, w, seq)[-1]
        if temperature <= 0 or topk == 1:
            top = torch.topk(logits, 2).values
            if doubtful is None and float(top[0] - top[1]) < margin:
                doubtful = i
        tok = plain_sample(logits, temperature, topk, topp, uniform_for(seed, len(seq)))
        out.append(tok); seq.append(tok)
    return out, doubtful


@pytest.fixture(scope="module")
def models(tiny_models):
    from infinicore_infer_b200.jiuge import JiugeForCauslLM
    cache = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in cache:
            cache[key] = JiugeForCauslLM(tiny_models[name][0], dtype=dtype, max_batch=8, **kw)
        return cache[key]
    return get


def assert_greedy(cfg, w, prompt, got, margin):
    """Every generated token is the plain implementation's choice for the sequence so far, or,
    where the plain logits of two tokens are closer than ``margin``, one of those."""
    seq = list(prompt)
    exact = 0
    for tok in got:
        logits = plain_forward(cfg, w, seq)[-1]
        best = float(logits.max())
        assert float(logits[tok]) >= best - margin, (len(seq), tok, int(logits.argmax()), best - float(logits[tok]))
        exact += int(tok == int(logits.argmax()))
        seq.append(tok)
    return exact


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_entry_point(tiny_models, models, name, dtype):
    _, cfg, w = tiny_models[name]
    model = models(name, dtype)
    model.eos_token_id = []
    for i, n in enumerate((5, 11, 17)):                 # the prompt lengths of the tiny-A workload
        prompt = random_tokens(500 + i, n, cfg["vocab_size"])
        scale = float(plain_forward(cfg, w, prompt).abs().max())
        got, avg_ms = model.generate(prompt, 8, verbose=False)
        assert len(got) == 8 and avg_ms >= 0.0
        if dtype == "float32":
            assert got == plain_generate(cfg, w, prompt, 8)[0], (name, n)
        else:       # bfloat16 may pick the other of two logits closer than twice its error bound
            assert assert_greedy(cfg, w, prompt, got, margin=2 * 2.5e-2 * scale) >= 6
    assert not model.engine.cache.lengths               # every cache handle was dropped


def test_tiny_a_workload_three_requests_eight_greedy_steps(tiny_models, models):
    _, cfg, w = tiny_models["A"]
    model = models("A", "float32")
    prompts = [random_tokens(600 + i, n, cfg["vocab_size"]) for i, n in enumerate((5, 11, 17))]
    got = model.generate_batch(prompts, max_new_tokens=8)
    eos = set(model.eos_token_id)
    for p, g in zip(prompts, got):
        want, _ = plain_generate(cfg, w, p, 8)
        if eos & set(want):
            want = want[:min(want.index(e) for e in eos if e in want) + 1]
        assert g == want


def test_tiny_b_workload_portions_mixed_with_decoding_at_temperature(tiny_models):
    """Four requests with prompts of 1/7/23/40 tokens, 9-token portions mixed with decoded tokens,
    temperature 0.8 with a fixed seed: the same tokens as the plain implementation, and the same
    whatever the portion size and the token budget."""
    from infinicore_infer_b200.jiuge import JiugeForCauslLM
    folder, cfg, w = tiny_models["B"]
    prompts = [random_tokens(700 + i, n, cfg["vocab_size"]) for i, n in enumerate((1, 7, 23, 40))]
    wants = [plain_generate(cfg, w, p, 10, temperature=0.8, seed=1234)[0] for p in prompts]
    outs = []
    for chunk, budget in ((9, 16), (512, 8192), (2, 7)):
        model = JiugeForCauslLM(folder, dtype="float32", max_batch=4, chunk_size=chunk, max_tokens_per_step=budget)
        reqs = [model.generator.submit(p, max_new_tokens=10, temperature=0.8, seed=1234, eos_token_ids=())
                for p in prompts]
        steps = 0
        while model.generator.scheduler.has_work():
            model.generator.step(); steps += 1
        outs.append([r.generated for r in reqs])
        if chunk == 9:
            assert model.generator.scheduler.counters["steps"] > 10 + 4     # prompts really were cut
    assert outs[0] == wants
    assert outs[1] == outs[0] and outs[2] == outs[0]


def test_sampling_is_reproducible_and_depends_on_the_seed(tiny_models, models):
    _, cfg, _ = tiny_models["B"]
    model = models("B", "bfloat16")
    prompt = random_tokens(800, 12, cfg["vocab_size"])
    kw = dict(max_new_tokens=12, temperature=6.0)         # hot enough that many tokens are likely
    a = model.generate_batch([prompt, prompt], seed=7, **kw)
    b = model.generate_batch([prompt], seed=7, **kw)
    c = model.generate_batch([prompt], seed=8, **kw)
    assert a[0] == a[1] == b[0]
    assert c[0] != b[0] and len(set(b[0])) > 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_under_page_pressure_preempts_and_still_matches(tiny_models, dtype):
    """A pool too small for three growing requests: the youngest is preempted and later recomputed.  float32: the
    tokens are the plain implementation's.  bfloat16 (the native runner, captured decode steps): every token is the
    plain choice for the sequence so far or within the error bound of it (a recomputed request meets its old positions
    through the prefill kernels instead of the decode kernels, so tokens need not equal those of an undisturbed run)."""
    from infinicore_infer_b200.jiuge import JiugeForCauslLM
    folder, cfg, w = tiny_models["A"]
    model = JiugeForCauslLM(folder, dtype=dtype, max_batch=4, cache_tokens=96, chunk_size=16)
    prompts = [random_tokens(900 + i, n, cfg["vocab_size"]) for i, n in enumerate((20, 25, 30))]
    got = model.generator.generate(prompts, max_new_tokens=24, eos_token_ids=())
    assert model.generator.scheduler.counters["preemptions"] >= 1
    if dtype == "float32":
        for p, g in zip(prompts, got):
            assert g == plain_generate(cfg, w, p, 24)[0]
    else:
        assert model.engine.runner is not None
        for p, g in zip(prompts, got):
            scale = float(plain_forward(cfg, w, p).abs().max())
            assert len(g) == 24 and assert_greedy(cfg, w, p, g, margin=2 * 2.5e-2 * scale) >= 18
    assert all(gr.pool.in_use == 0 for gr in model.engine.cache.groups)


def test_round_by_round_with_tasks_and_the_cache_pool(tiny_models, models):
    """The reference's call pattern: InferTask + KVCachePool + batch_infer_one_round, with a second
    request that reuses the first one's cache at their common prefix."""
    from infinicore_infer_b200.tasks import InferTask, KVCachePool
    _, cfg, w = tiny_models["B"]
    model = models("B", "float32")
    pool = KVCachePool(model, max_caches=1)
    shared = random_tokens(1000, 14, cfg["vocab_size"])
    p1 = shared + random_tokens(1001, 5, cfg["vocab_size"])
    p2 = shared + random_tokens(1002, 9, cfg["vocab_size"])

    def run(prompt, steps):
        task = InferTask(0, list(prompt), model.max_context_len(), 0.0, 1, 1.0, [])
        pool.acquire_sync(task)
        start = task.pos
        out = []
        for _ in range(steps):
            tok = model.batch_infer_one_round([task])[0]
            out.append(tok)
            task.next(tok)
        pool.release_sync(task)
        return out, start

    o1, s1 = run(p1, 6)
    o2, s2 = run(p2, 6)
    assert s1 == 0 and s2 == 14                         # the second request starts at the shared prefix
    assert o1 == plain_generate(cfg, w, p1, 6)[0] and o2 == plain_generate(cfg, w, p2, 6)[0]
    pool.finalize()
    assert not model.engine.cache.lengths


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_rounds_run_from_what_the_round_before_prepared(tiny_models, dtype):
    """In a loop of ``batch_infer_one_round`` a decode step prepares the next one (pages, metadata) while the device
    runs; the tokens are the plain implementation's all the same, and when the next call is another step than the
    one prepared, the pages taken ahead are back before it is planned."""
    from infinicore_infer_b200.jiuge import JiugeForCauslLM
    from infinicore_infer_b200.tasks import InferTask, KVCache
    folder, cfg, w = tiny_models["A"]
    model = JiugeForCauslLM(folder, dtype=dtype, max_batch=4, page_size=8, num_pages=16)
    eng = model.engine
    prompts = [random_tokens(2100 + i, n, cfg["vocab_size"]) for i, n in enumerate((7, 15))]
    tasks = []
    for i, p in enumerate(prompts):
        t = InferTask(i, list(p), model.max_context_len(), 0.0, 1, 1.0, [])
        t.bind_kvcache(KVCache(model))
        tasks.append(t)
    outs = [[], []]
    for _ in range(12):                                   # 15 + 12 crosses page edges of 8 for both requests
        for t, o, tok in zip(tasks, outs, model.batch_infer_one_round(tasks)):
            o.append(tok)
            t.next(tok)
    assert eng.staged_steps >= 9                          # all but the prompts' step, the first decode step and its capture
    margin = 0.0 if dtype == "float32" else 0.05
    for p, o in zip(prompts, outs):
        assert_greedy(cfg, w, p, o, margin)
    eng.cache.check_invariants()
    # the step that was prepared is not the one that comes: one request alone, then a new prompt beside it
    in_use = lambda: [g.pool.in_use for g in eng.cache.groups]
    before = in_use()
    tok = model.batch_infer_one_round(tasks[:1])[0]
    assert_greedy(cfg, w, prompts[0] + outs[0], [tok], margin)
    tasks[0].next(tok)
    eng.cache.check_invariants()
    third = InferTask(2, random_tokens(2103, 9, cfg["vocab_size"]), model.max_context_len(), 0.0, 1, 1.0, [])
    third.bind_kvcache(KVCache(model))
    toks = model.batch_infer_one_round([tasks[0], third])
    assert_greedy(cfg, w, list(third.tokens), [toks[1]], margin)
    for t in tasks + [third]:
        t.kvcache().drop(model)
    assert in_use() == [0] * len(eng.cache.groups) and before != in_use()
    eng.check()


def test_perplexity_matches_the_plain_implementation(tiny_models, models):
    _, cfg, w = tiny_models["C"]
    model = models("C", "float32")
    seqs = [random_tokens(1100 + i, n, cfg["vocab_size"]) for i, n in enumerate((9, 30, 17))]
    nll, total = 0.0, 0
    for s in seqs:
        logp = torch.log_softmax(plain_forward(cfg, w, s[:-1]), -1)
        nll += float(-logp[torch.arange(len(s) - 1), torch.tensor(s[1:])].sum()); total += len(s) - 1
    want = float(np.exp(nll / total))
    assert abs(model.perplexity(seqs, batch_size=2) - want) <= 1e-4 * want


def test_device_flags_of_the_reference_are_refused_except_nvidia(tiny_models):
    from infinicore_infer_b200.jiuge import DeviceType, JiugeForCauslLM, test as cli
    with pytest.raises(ValueError, match="sm_100a"):
        JiugeForCauslLM(tiny_models["A"][0], DeviceType.DEVICE_TYPE_ASCEND)
    with pytest.raises(ValueError, match="one device"):
        JiugeForCauslLM(tiny_models["A"][0], DeviceType.DEVICE_TYPE_NVIDIA, ndev=2)
    assert cli([]) == 1 and cli(["--cpu", tiny_models["A"][0]]) == 1


def test_command_line(tiny_models):
    folder = tiny_models["A"][0]
    proc = subprocess.run([sys.executable, "-m", "infinicore_infer_b200.jiuge", "--nvidia", folder,
                           "--prompt-ids", "5,17,3,99", "--max-steps", "6", "--dtype", "float32"],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "Time per step" in proc.stdout and "Model destroyed" in proc.stdout


def test_command_line_runs_the_tiny_b_workload_through_the_scheduler(tmp_path):
    """``--random tiny-B`` with four prompts of 1/7/23/40 tokens, portions of 9 beside decoded tokens, pages of 8,
    temperature 0.8 with a fixed seed: the printed tokens are the plain implementation's."""
    import re
    from infinicore_infer_b200.config import PRESETS, MiniCPMConfig
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    preset = PRESETS["tiny-B"]
    proc = subprocess.run([sys.executable, "-m", "infinicore_infer_b200.jiuge", "--nvidia", "--random", "tiny-B", "--seed", "1",
                           "--prompt-lens", "1,7,23,40", "--chunk-size", "9", "--page-size", "8", "--num-pages", "40",
                           "--max-batch", "4", "--max-tokens-per-step", "16", "--temperature", "0.8", "--topk", "0",
                           "--sample-seed", "1234", "--max-steps", "10", "--dtype", "float32"],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = {int(m.group(1)): [int(t) for t in m.group(2).split()] for m in re.finditer(r"request (\d+): ([\d ]*)", proc.stdout)}
    assert sorted(got) == [0, 1, 2, 3]
    steps = int(re.search(r"(\d+) steps", proc.stdout).group(1))
    assert steps > 10 + 4                                # the prompts really were cut into portions
    cfg = MiniCPMConfig.from_dict(preset.config)
    write_model_folder(cfg, str(tmp_path), seed=1, std=preset.std, norm_std=preset.norm_std)
    w = {n: read_tensor(i).float() for n, i in index_directory(str(tmp_path)).items()}
    eos = set(cfg.eos_token_id)
    for k, n in enumerate((1, 7, 23, 40)):
        prompt = torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(1 + k)).tolist()
        want, _ = plain_generate(cfg.to_dict(), w, prompt, 10, temperature=0.8, seed=1234)
        if eos & set(want):
            want = want[:min(want.index(e) for e in eos if e in want) + 1]
        assert got[k] == want, k


def test_command_line_refuses_a_folder_together_with_a_random_model(tiny_models):
    from infinicore_infer_b200.jiuge import test as cli
    assert cli(["--nvidia", tiny_models["A"][0], "--random", "tiny-A"]) == 1
    assert cli(["--nvidia"]) == 1
