"""The Python entry point and the command line, in the reference's manner.

    python -m infinicore_infer_b200.jiuge --nvidia <path/to/model_dir> [n_device] [options]

``JiugeForCauslLM`` (the reference's spelling; ``JiugeForCausalLM`` is the same class) mirrors
scripts/jiuge.py:396-643: built from a model folder, it offers ``max_context_len``,
``create_kv_cache`` / ``drop_kv_cache``, ``batch_infer_one_round(tasks)``, ``generate``,
``perplexity`` and ``destroy_model_instance``.  Differences that a user of the reference
meets: the device is an sm_100a GPU (the other device flags are refused, as is more than one
device); prompts may be given as token ids, so no tokenizer is needed; sampling is
reproducible (``seed``); ``dtype`` selects bfloat16 or a true float32 path.
"""
from __future__ import annotations

import argparse
import math
import sys
import time
from typing import List, Optional, Sequence

import torch

from .engine import Engine, Generator, StepEntry
from .sampling import Sampler, SamplingParams
from .tasks import InferTask, KVCache, KVCachePool


class DeviceType:
    """The reference's device enumeration (scripts/libinfinicore_infer.py:29-36); one is served."""
    DEVICE_TYPE_CPU = 0
    DEVICE_TYPE_NVIDIA = 1
    DEVICE_TYPE_CAMBRICON = 2
    DEVICE_TYPE_ASCEND = 3
    DEVICE_TYPE_METAX = 4
    DEVICE_TYPE_MOORE = 5
    DEVICE_TYPE_ILUVATAR = 6


_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32}


class JiugeForCauslLM:
    def __init__(self, model_dir_path, device=DeviceType.DEVICE_TYPE_NVIDIA, ndev=1, max_tokens=None,
                 dtype="bfloat16", device_id=0, cache_tokens: Optional[int] = None, page_size: int = 16,
                 max_batch: int = 64, max_tokens_per_step: int = 8192, chunk_size: int = 512,
                 use_graphs: bool = True):
        if device != DeviceType.DEVICE_TYPE_NVIDIA:
            raise ValueError("this engine runs on NVIDIA sm_100a only; pass DeviceType.DEVICE_TYPE_NVIDIA")
        if ndev != 1:
            raise ValueError("this engine runs on one device; ndev must be 1")
        t0 = time.time()
        print("Loading model weights to device...")
        dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        from .config import read_config
        ctx = read_config(model_dir_path, max_tokens=max_tokens).max_position_embeddings
        self.engine = Engine.from_folder(
            model_dir_path, dtype=dt, device=f"cuda:{device_id}", max_tokens=max_tokens,
            cache_tokens=cache_tokens or max(ctx * min(max_batch, 4), 4096), page_size=page_size,
            max_requests=max_batch, max_step_tokens=max_tokens_per_step, use_graphs=use_graphs)
        self._attach(self.engine, model_dir_path, max_batch, max_tokens_per_step, chunk_size)
        print(f"Time used: {time.time() - t0:.3f}s")

    def _attach(self, engine: Engine, model_dir_path, max_batch, max_tokens_per_step, chunk_size) -> None:
        self.engine = engine
        self.config = getattr(engine, "config", None)
        self.eos_token_id = list(engine.spec.eos_token_ids)
        self.generator = Generator(engine, max_batch=max_batch, max_tokens_per_step=max_tokens_per_step,
                                   chunk_size=chunk_size)
        self.sampler = Sampler(engine.device)
        self.model_dir_path = model_dir_path
        self._tokenizer = None
        self._next_cache = 0
        self.sample_seed = 0

    @classmethod
    def from_engine(cls, engine: Engine, max_batch: Optional[int] = None, max_tokens_per_step: Optional[int] = None,
                    chunk_size: int = 512) -> "JiugeForCauslLM":
        """The same entry point over an engine that exists already (e.g. one with random weights
        made on the device, for shapes whose checkpoint would be gigabytes on disk)."""
        self = cls.__new__(cls)
        self._attach(engine, None, max_batch or engine.max_requests,
                     max_tokens_per_step or engine.max_step_tokens, chunk_size)
        return self

    # ---- the reference's methods ------------------------------------------------------------------
    def max_context_len(self) -> int:
        return self.engine.spec.max_positions

    def create_kv_cache(self):
        """A new cache handle: a request of the paged cache that holds nothing yet."""
        handle = f"kv{self._next_cache}"
        self._next_cache += 1
        self.engine.begin(handle)
        return handle

    def drop_kv_cache(self, kv_cache) -> None:
        if self.engine.cache.is_live(kv_cache):
            self.engine.end(kv_cache)

    def _entries(self, tasks: Sequence[InferTask], want_all: bool = False) -> List[StepEntry]:
        entries = []
        for t in tasks:
            handle = t.kvcache().data()
            if self.engine.position(handle) != t.pos:
                # the task starts at a prefix of what the handle holds (reuse by the pool)
                self.engine.cache.truncate(handle, t.pos)
            n = len(t.tokens)
            entries.append(StepEntry(handle, list(t.tokens), list(range(n)) if want_all else [n - 1]))
        return entries

    def batch_infer_one_round(self, tasks: List[InferTask]) -> List[int]:
        """One step over the tasks' pending tokens; one sampled token per task (scripts/jiuge.py:529-537)."""
        logits = self.engine.step(self._entries(tasks))
        params = [SamplingParams(t.temperature, t.topk, t.topp, getattr(t, "seed", self.sample_seed)) for t in tasks]
        return self.sampler.sample(logits, params, [t.pos + len(t.tokens) for t in tasks])

    def forward_batch(self, tasks: List[InferTask]) -> torch.Tensor:
        """Logits of every fed row, float32 on the device (the reference's ``forwardBatch``)."""
        return self.engine.step(self._entries(tasks, want_all=True))

    def generate(self, input_content, max_steps, topp_=1.0, topk_=1, temperature_=1.0, seed=0, verbose=True):
        """Generate up to ``max_steps`` tokens after the prompt.  ``input_content`` is a list of
        token ids, or a string if the model folder has a tokenizer.  Returns (output, average
        milliseconds per decode step), the prompt's step excluded as in scripts/jiuge.py:578-583."""
        as_text = isinstance(input_content, str)
        tokens = self._encode(input_content) if as_text else list(input_content)
        task = InferTask(0, tokens, self.max_context_len(), temperature_, topk_, topp_, self.eos_token_id)
        task.seed = seed
        task.bind_kvcache(KVCache(self))
        out: List[int] = []
        total = 0.0
        steps = 0
        for i in range(max_steps):
            t0 = time.time()
            tok = self.batch_infer_one_round([task])[0]
            dt = time.time() - t0
            steps += 1
            out.append(tok)
            if verbose:
                print(self._decode([tok]) if as_text else tok, end="" if as_text else " ", flush=True)
            if tok in self.eos_token_id:
                break
            task.next(tok)
            if task.finish_reason is not None:
                break
            if i > 0:
                total += dt
        if verbose:
            print("\n")
        avg = total * 1000 / (steps - 1) if steps > 1 else 0.0
        if verbose:
            print(f"Time per step: {avg:.3f}ms")
        task.kvcache().drop(self)
        return (self._decode(out) if as_text else out), avg

    def perplexity(self, test_sequences: List[Sequence[int]], batch_size=10) -> float:
        """exp(mean negative log-likelihood) of the sequences' next tokens (scripts/jiuge.py:588-639)."""
        nll, total = 0.0, 0
        for i in range(0, len(test_sequences), batch_size):
            batch = test_sequences[i:i + batch_size]
            tasks, caches = [], []
            for j, seq in enumerate(batch):
                t = InferTask(j, list(seq[:-1]), self.max_context_len(), 1.0, 1, 1.0, self.eos_token_id)
                kv = KVCache(self)
                t.bind_kvcache(kv)
                tasks.append(t); caches.append(kv)
            logits = self.forward_batch(tasks)
            target = torch.tensor([tok for seq in batch for tok in seq[1:]], device=logits.device)
            logp = torch.log_softmax(logits.float(), dim=-1)
            nll += float(-logp[torch.arange(len(target), device=logits.device), target].sum())
            total += len(target)
            for kv in caches:
                kv.drop(self)
        return math.exp(nll / total)

    def destroy_model_instance(self) -> None:
        self.engine = None
        self.generator = None
        torch.cuda.empty_cache()
        print("Model destroyed")

    # ---- generation of many requests through the scheduler ------------------------------------------
    def generate_batch(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0,
                       topk: int = 0, topp: float = 1.0, seed: int = 0) -> List[List[int]]:
        """Token ids in, token ids out, for many prompts at once: admission, portions of prompts under
        the token budget, batched decoding and freeing are the scheduler's."""
        return self.generator.generate(prompts, max_new_tokens=max_new_tokens, temperature=temperature,
                                       topk=topk, topp=topp, seed=seed)

    # ---- text, when the folder has a tokenizer -------------------------------------------------------
    def _tok(self):
        if self._tokenizer is None:
            try:
                import transformers
                self._tokenizer = transformers.AutoTokenizer.from_pretrained(self.model_dir_path, trust_remote_code=True)
            except Exception as e:        # noqa: BLE001 - any failure means: no tokenizer in this folder
                raise ValueError(f"no usable tokenizer in {self.model_dir_path} ({e}); pass token ids instead") from None
        return self._tokenizer

    def _encode(self, text: str) -> List[int]:
        tok = self._tok()
        try:
            text = tok.apply_chat_template(conversation=[{"role": "user", "content": text}],
                                           add_generation_prompt=True, tokenize=False)
        except Exception:                 # noqa: BLE001 - a tokenizer without a chat template
            pass
        return tok.encode(text)

    def _decode(self, ids: List[int]) -> str:
        return self._tok().decode(ids)


JiugeForCausalLM = JiugeForCauslLM

_DEVICE_FLAGS = {"--cpu": DeviceType.DEVICE_TYPE_CPU, "--nvidia": DeviceType.DEVICE_TYPE_NVIDIA,
                 "--cambricon": DeviceType.DEVICE_TYPE_CAMBRICON, "--ascend": DeviceType.DEVICE_TYPE_ASCEND,
                 "--metax": DeviceType.DEVICE_TYPE_METAX, "--moore": DeviceType.DEVICE_TYPE_MOORE,
                 "--iluvatar": DeviceType.DEVICE_TYPE_ILUVATAR}


def test(argv=None) -> int:
    """``jiuge.py --nvidia <model_dir> [n_device]`` as in scripts/jiuge.py:646-677, plus options."""
    argv = list(sys.argv[1:] if argv is None else argv)
    usage = ("Usage: python -m infinicore_infer_b200.jiuge [--cpu | --nvidia | --cambricon | --ascend | --metax | "
             "--moore | --iluvatar] <path/to/model_dir> [n_device] [--dtype bfloat16|float32] "
             "[--prompt-ids 1,2,3 | --prompt TEXT | --prompt-len N] [--max-steps N] [--temperature F] "
             "[--topk N] [--topp F] [--seed N] [--max-tokens N] [--requests N]")
    if len(argv) < 2 or argv[0] not in _DEVICE_FLAGS:
        print(usage)
        return 1
    device = _DEVICE_FLAGS[argv[0]]
    if device != DeviceType.DEVICE_TYPE_NVIDIA:
        print(f"{argv[0]}: this engine is written for NVIDIA sm_100a only; use --nvidia")
        return 1
    ap = argparse.ArgumentParser(prog="jiuge", usage=usage)
    ap.add_argument("model_dir")
    ap.add_argument("n_device", nargs="?", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16", choices=sorted(_DTYPES))
    ap.add_argument("--prompt", default=None, help="text (needs a tokenizer in the model folder)")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    ap.add_argument("--prompt-len", type=int, default=16, help="random prompt of this length if none is given")
    ap.add_argument("--max-steps", type=int, default=500, help="tokens to generate (scripts/jiuge.py:676 runs 500)")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--topk", type=int, default=1)
    ap.add_argument("--topp", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-tokens", type=int, default=None, help="context length override (the reference's max_tokens)")
    ap.add_argument("--requests", type=int, default=1, help="generate for this many copies of the prompt at once")
    args = ap.parse_args(argv[1:])
    if args.n_device != 1:
        print("n_device must be 1: this engine runs on one GPU")
        return 1
    model = JiugeForCauslLM(args.model_dir, device, args.n_device, max_tokens=args.max_tokens, dtype=args.dtype)
    if args.prompt is not None:
        prompt = args.prompt
    elif args.prompt_ids:
        prompt = [int(t) for t in args.prompt_ids.split(",")]
    else:
        g = torch.Generator().manual_seed(args.seed)
        prompt = torch.randint(0, model.engine.spec.vocab_size, (args.prompt_len,), generator=g).tolist()
    if args.requests > 1:
        ids = model._encode(prompt) if isinstance(prompt, str) else prompt
        t0 = time.time()
        outs = model.generate_batch([ids] * args.requests, max_new_tokens=args.max_steps,
                                    temperature=0.0 if args.topk == 1 else args.temperature,
                                    topk=args.topk, topp=args.topp, seed=args.seed)
        dt = time.time() - t0
        n = sum(len(o) for o in outs)
        print(outs[0])
        print(f"{n} tokens for {args.requests} requests in {dt:.3f}s: {n / dt:.1f} tok/s")
    else:
        model.generate(prompt, args.max_steps, topp_=args.topp, topk_=args.topk, temperature_=args.temperature,
                       seed=args.seed)
    model.destroy_model_instance()
    return 0


if __name__ == "__main__":
    sys.exit(test())
