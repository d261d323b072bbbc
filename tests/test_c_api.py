"""The C interface (csrc/model_api.h) through its ctypes wrapper: the same logits as the plain implementation
however a request is cut into batches, the same tokens as the Python engine, and a page pool that loses nothing."""
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

from conftest import random_tokens
from test_replay import TOL, expected, make_engine

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "infinicore-infer_b200", "csrc", "model_api.h")


def test_the_header_is_plain_c(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "use.c"
    src.write_text(f'#include "{HEADER}"\nint main(void) {{ JkModelMeta m; JkModelOptions o; (void)m; (void)o; return 0; }}\n')
    subprocess.run([cc, "-std=c99", "-Wall", "-Werror", "-fsyntax-only", str(src)], check=True)


@pytest.mark.gpu
def test_a_c_program_runs_the_engine_without_python(tmp_path):
    """tests/c_api_program.c, compiled by the C compiler against csrc/model_api.h and linked with the runner's shared
    object only: it finds the kernel modules in the build folder itself, runs a prompt whole and in pieces, generates
    a few tokens, and exits 0 if the two ways of cutting agree and no page was lost."""
    from infinicore_infer_b200.kernels import build
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    for module in build.MODULES:
        build.build(module)
    folder = build.build_dir()
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / "prog")
    subprocess.run([cc, "-std=c99", "-Wall", "-I", os.path.dirname(HEADER), os.path.join(here, "c_api_program.c"), "-o", exe,
                    "-L", folder, "-ljk_runner", f"-Wl,-rpath,{folder}", "-lm"], check=True)
    run = subprocess.run([exe, folder], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "greedy:" in run.stdout and "largest difference" in run.stdout


def native(models, name, **kw):
    from infinicore_infer_b200.engine.native_model import NativeModel
    kw.setdefault("page_size", 16)
    kw.setdefault("cache_tokens", 1024)
    kw.setdefault("max_step_tokens", 1024)
    return NativeModel.from_folder(models[name][0], **kw)


def close(want, got, what):
    scale = np.abs(want).max()
    err = np.abs(got.astype(np.float64) - want).max(axis=-1)
    bad = np.nonzero(err > TOL["bfloat16"] * scale)[0]
    assert bad.size == 0, f"{what}: first wrong position {bad[0]}: error {err[bad[0]]:.3e} > {TOL['bfloat16'] * scale:.3e}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])      # C: sizes outside the fast kernels; E: q/k/v biases
def test_forward_batch_whole_in_portions_and_token_by_token(tiny_models, name):
    m = native(tiny_models, name)
    toks, want = expected(tiny_models, name, 700, 200)
    pool = m.free_pages
    # whole
    c = m.create_kv_cache()
    close(want, m.forward_batch([toks], [0], [c]), f"{name} whole")
    m.drop_kv_cache(c)
    assert m.free_pages == pool
    # portions of changing size (several tiles, ragged ends, down to two tokens), then single tokens
    c = m.create_kv_cache()
    pos, rows = 0, []
    for n in (130, 2, 17, 9, 3) + (1,) * 39:
        rows.append(m.forward_batch([toks[pos: pos + n]], [pos], [c]))
        pos += n
    assert pos == len(toks)
    close(want, np.concatenate(rows), f"{name} portions")
    m.drop_kv_cache(c)
    assert m.free_pages == pool
    m.close()


@pytest.mark.gpu
def test_mixed_batches_in_a_pool_so_small_that_pages_are_used_again(tiny_models):
    name = "D"
    m = native(tiny_models, name, cache_tokens=224)          # 14 pages of 16
    lens = {"a": 70, "b": 33, "c": 90, "d": 48, "e": 61}
    toks, wants = {}, {}
    for i, (r, n) in enumerate(lens.items()):
        toks[r], wants[r] = expected(tiny_models, name, 720 + i, n)
    plan = [{"a": 40}, {"a": 2, "b": 30}, {"a": 28, "b": 3}, {"c": 50}, {"c": 1, "d": 20}, {"c": 39, "d": 28}, {"e": 61}]
    ends = {2: ["a", "b"], 5: ["c", "d"], 6: ["e"]}
    caches, done, got = {}, {r: 0 for r in lens}, {r: [] for r in lens}
    pool = m.free_pages
    for step, batch in enumerate(plan):
        reqs = list(batch)
        for r in reqs:
            if r not in caches:
                caches[r] = m.create_kv_cache()
        out = m.forward_batch([toks[r][done[r]: done[r] + batch[r]] for r in reqs], [done[r] for r in reqs],
                              [caches[r] for r in reqs])
        row = 0
        for r in reqs:
            got[r].append(out[row: row + batch[r]])
            row += batch[r]
            done[r] += batch[r]
        for r in ends.get(step, []):
            m.drop_kv_cache(caches.pop(r))
    assert m.free_pages == pool and done == lens
    for r in lens:
        close(wants[r], np.concatenate(got[r]), f"mixed request {r}")
    m.close()


@pytest.mark.gpu
def test_a_batch_that_does_not_fit_takes_no_page(tiny_models):
    from infinicore_infer_b200.engine.native_model import NativeModelError
    m = native(tiny_models, "A", cache_tokens=64)            # 4 pages
    toks = random_tokens(5, 80, 256)
    a, b = m.create_kv_cache(), m.create_kv_cache()
    m.forward_batch([toks[:40]], [0], [a])
    assert m.free_pages == 1
    with pytest.raises(NativeModelError, match="cache pages"):
        m.forward_batch([toks[40:48], toks[:20]], [40, 0], [a, b])       # a needs none, b needs two
    assert m.free_pages == 1
    with pytest.raises(NativeModelError, match="starts at position"):
        m.forward_batch([toks[:4]], [70], [b])
    with pytest.raises(NativeModelError, match="share a cache"):
        m.forward_batch([toks[:4], toks[:4]], [40, 40], [a, a])
    with pytest.raises(NativeModelError, match="outside the vocabulary"):
        m.forward_batch([[256]], [40], [a])
    m.forward_batch([toks[:16]], [0], [b])
    assert m.free_pages == 0
    m.drop_kv_cache(a)
    m.drop_kv_cache(b)
    assert m.free_pages == 4
    m.close()


@pytest.mark.gpu
def test_a_duplicated_cache_continues_like_the_original(tiny_models):
    name = "B"
    m = native(tiny_models, name)
    toks, want = expected(tiny_models, name, 730, 90)
    a = m.create_kv_cache()
    m.forward_batch([toks[:50]], [0], [a])
    b = m.duplicate_kv_cache(a, 37)                           # a page's middle: the copy holds the page's rest too
    other = random_tokens(6, 13, 384)
    m.forward_batch([other], [37], [b])                       # overwrite positions 37.. of the copy only
    rest_a = m.forward_batch([toks[50:]], [50], [a])
    close(want[50:], rest_a, "the original after its copy was written")
    c = m.duplicate_kv_cache(a, 90)
    again = m.forward_batch([toks[37:]], [37], [m.duplicate_kv_cache(a, 37)])
    close(want[37:], again, "a copy of the first 37 tokens, continued")
    last = m.forward_batch([toks[89:]], [89], [c])
    close(want[89:], last, "a whole copy, last token again")
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["A", "D"])
def test_infer_batch_generates_what_the_engine_generates(tiny_models, name):
    from infinicore_infer_b200.engine import Generator
    vocab = tiny_models[name][1]["vocab_size"]
    prompts = [random_tokens(740 + i, n, vocab) for i, n in enumerate((23, 5, 41))]
    new = 12
    sampling = [dict(temperature=0.0, topk=0, topp=1.0, seed=0), dict(temperature=0.9, topk=20, topp=0.9, seed=11),
                dict(temperature=1.3, topk=0, topp=1.0, seed=5)]
    gen = Generator(make_engine(tiny_models[name][0], "bfloat16", 1024))
    reqs = [gen.submit(p, max_new_tokens=new, eos_token_ids=(), **s) for p, s in zip(prompts, sampling)]
    gen.run()
    want = [r.generated for r in reqs]

    m = native(tiny_models, name)
    caches = [m.create_kv_cache() for _ in prompts]
    seqs = [list(p) for p in prompts]
    par = dict(temperature=[s["temperature"] for s in sampling], topk=[s["topk"] for s in sampling],
               topp=[s["topp"] for s in sampling], seeds=[s["seed"] for s in sampling])
    out = m.infer_batch(prompts, [0, 0, 0], caches, **par)
    got = [[t] for t in out]
    for _ in range(new - 1):
        pos = [len(s) + len(g) - 1 for s, g in zip(seqs, got)]
        out = m.infer_batch([[g[-1]] for g in got], pos, caches, **par)
        for g, t in zip(got, out):
            g.append(t)
    assert m.last_launches > 0
    # greedy: the same kernels on the same numbers; drawn tokens: the same uniform numbers by (seed, position)
    assert got == want
    m.close()
