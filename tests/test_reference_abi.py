"""The reference's own, unmodified Python side driving this engine through the reference's C interface.

``csrc/reference_abi.cu`` gives this engine the symbols that scripts/libinfinicore_infer.py opens
(``createJiugeModel``, ``createKVCache``, ``dropKVCache``, ``inferBatch``, ``forwardBatch``, ``destroyJiugeModel``).
Here ``$INFINI_ROOT/lib/libinfinicore_infer.so`` is a link to this engine's library, scripts/jiuge.py is imported as
it stands, its ``JiugeMetaFromLlama`` and ``JiugeWeightsImpl`` read a tiny random model (permuting query and key rows,
folding the scales into the weights), its ``JiugeBatchedTask`` marshals the batches, and the logits and tokens that
come back are held against the plain implementation.  What this pins that nothing else does: that the reference's
packing, taken as the reference makes it, means the same model as the checkpoint does to this engine.
Skips where the reference's scripts are not on the machine.
"""
import os
from ctypes import POINTER, byref, c_int, c_uint

import numpy as np
import pytest
import torch

from conftest import TINY, random_tokens
from plain_minicpm import plain_forward
import reference_scripts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(tmp_path_factory):
    if reference_scripts.scripts_dir() is None:
        pytest.skip("the reference's scripts are not on this machine")
    if "libinfinicore_infer" in __import__("sys").modules:
        pytest.skip("the reference's binding is already loaded over another library in this process")
    from infinicore_infer_b200.kernels import build
    for module in build.MODULES:              # the library finds the kernel modules beside itself
        build.build(module)
    root = str(tmp_path_factory.mktemp("infini_root"))
    os.makedirs(os.path.join(root, "lib"))
    os.symlink(build.library_path("runner"), os.path.join(root, "lib", "libinfinicore_infer.so"))
    try:
        (jiuge,) = reference_scripts.import_reference(root)
    except Exception as e:       # noqa: BLE001
        pytest.skip(f"the reference's scripts do not import here: {e}")
    return jiuge


class Harness:
    """What scripts/jiuge.py's JiugeForCauslLM does after loading, without its tokenizer: create the model from the
    reference's meta and weights, and its methods that the reference's request objects call."""

    def __init__(self, jiuge, cfg, state):
        self.jiuge = jiuge
        self.meta = jiuge.JiugeMetaFromLlama(cfg, dtype=torch.bfloat16)
        self.weights = jiuge.JiugeWeightsImpl(self.meta, jiuge.LlamaWeightsNaming(), state, torch_dt_mat=torch.bfloat16,
                                              torch_dt_norm=torch.float32)
        dev_ids = (c_int * 1)(0)
        self.model_instance = jiuge.create_jiuge_model(byref(self.meta), byref(self.weights), jiuge.DeviceType.DEVICE_TYPE_NVIDIA, 1, dev_ids)
        assert self.model_instance, "createJiugeModel returned null"

    def max_context_len(self):
        return self.meta.dctx

    def create_kv_cache(self):
        return self.jiuge.create_kv_cache(self.model_instance)

    def drop_kv_cache(self, kv):
        self.jiuge.drop_kv_cache(self.model_instance, kv)

    def forward(self, tasks):
        batch = self.jiuge.JiugeBatchedTask(tasks)
        logits = torch.zeros((batch.ntok, self.meta.dvoc), dtype=self.meta.torch_dtype_logits)
        self.jiuge.forward_batch(self.model_instance, batch.tokens, batch.ntok, batch.req_lens, batch.nreq, batch.req_pos,
                                 batch.kv_caches, logits.data_ptr())
        return logits.float().numpy()

    def infer(self, tasks):
        batch = self.jiuge.JiugeBatchedTask(tasks)
        out = (c_uint * len(tasks))()
        self.jiuge.infer_batch(self.model_instance, *batch.input_args(), out)
        return list(out)

    def close(self):
        self.jiuge.destroy_jiuge_model(self.model_instance)


@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_the_reference_s_python_drives_this_engine(ref, tiny_models, name):
    jiuge = ref
    _, cfg, w = tiny_models[name]
    state = {k: v.clone() for k, v in w.items()}          # float32 copies of the checkpoint's bfloat16 values
    model = Harness(jiuge, cfg, state)
    V = cfg["vocab_size"]
    toks_a, toks_b = random_tokens(81, 150, V), random_tokens(82, 37, V)
    want_a, want_b = plain_forward(cfg, w, toks_a).numpy(), plain_forward(cfg, w, toks_b).numpy()
    # the reference's request objects: a whole prompt beside another, then portions and single tokens of the first
    ta = jiuge.InferTask(0, list(toks_a[:100]), model.max_context_len(), 0.0, 1, 1.0, [])
    tb = jiuge.InferTask(1, list(toks_b), model.max_context_len(), 0.0, 1, 1.0, [])
    ta.bind_kvcache(jiuge.KVCache(model))
    tb.bind_kvcache(jiuge.KVCache(model))
    got = model.forward([ta, tb])
    # logits come back in bfloat16 (the reference's activation type): one more rounding than this engine's float32
    tol = 3e-2
    assert np.abs(got[:100] - want_a[:100]).max() <= tol * np.abs(want_a).max()
    assert np.abs(got[100:] - want_b).max() <= tol * np.abs(want_b).max()
    rows = []
    pos = 100
    for n in (30, 2, 1, 1, 16):
        ta.tokens, ta.pos = list(toks_a[pos:pos + n]), pos
        rows.append(model.forward([ta]))
        pos += n
    assert pos == 150
    assert np.abs(np.concatenate(rows) - want_a[100:]).max() <= tol * np.abs(want_a).max()
    # greedy generation through inferBatch, the reference's loop (scripts/jiuge.py:556-576): every token is the plain
    # choice for the sequence so far, or within the error bound of it
    prompt = random_tokens(83, 12, V)
    task = jiuge.InferTask(2, list(prompt), model.max_context_len(), 1.0, 1, 1.0, [])
    task.bind_kvcache(jiuge.KVCache(model))
    seq = list(prompt)
    for _ in range(8):
        tok = model.infer([task])[0]
        logits = plain_forward(cfg, w, seq)[-1]
        assert tok < V and float(logits[tok]) >= float(logits.max()) - 2 * 2.5e-2 * float(logits.abs().max()), (len(seq), tok)
        seq.append(tok)
        task.next(tok)
    for t in (ta, tb, task):
        t.kvcache().drop(model)
    model.close()
