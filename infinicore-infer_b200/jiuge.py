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


def _check_device(device, ndev) -> None:
    if device != DeviceType.DEVICE_TYPE_NVIDIA:
        raise ValueError("this engine runs on NVIDIA sm_100a only; pass DeviceType.DEVICE_TYPE_NVIDIA")
    if ndev != 1:
        raise ValueError("this engine runs on one device; ndev must be 1")


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class JiugeForCauslLM:
    def __init__(self, model_dir_path, device=DeviceType.DEVICE_TYPE_NVIDIA, ndev=1, max_tokens=None,
                 dtype="bfloat16", device_id=0, cache_tokens: Optional[int] = None, page_size: int = 16,
                 max_batch: int = 64, max_tokens_per_step: int = 8192, chunk_size: int = 512,
                 use_graphs: bool = True, num_pages: Optional[int] = None, strict_weights: bool = False):
        """``cache_tokens`` (or ``num_pages`` pages of ``page_size`` tokens) sizes the pool that all requests share;
        ``max_batch`` bounds the requests of a step, ``max_tokens_per_step`` its tokens, ``chunk_size`` a prompt's
        portion.  The first four arguments are the reference's (scripts/jiuge.py:397-399)."""
        _check_device(device, ndev)
        t0 = time.time()
        print("Loading model weights to device...")
        dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        from .config import read_config
        ctx = read_config(model_dir_path, max_tokens=max_tokens).max_position_embeddings
        if num_pages is not None:
            cache_tokens = num_pages * page_size
        self.engine = Engine.from_folder(
            model_dir_path, dtype=dt, device=f"cuda:{device_id}", max_tokens=max_tokens,
            cache_tokens=cache_tokens or max(ctx * min(max_batch, 4), 4096), page_size=page_size,
            max_requests=max_batch, max_step_tokens=max_tokens_per_step, use_graphs=use_graphs,
            strict_weights=strict_weights)
        self._attach(self.engine, model_dir_path, max_batch, max_tokens_per_step, chunk_size)
        print(f"Time used: {time.time() - t0:.3f}s")

    @classmethod
    def from_random(cls, preset: str, seed: int = 0, dtype="bfloat16", device_id: int = 0, max_tokens=None,
                    cache_tokens: Optional[int] = None, page_size: Optional[int] = None, num_pages: Optional[int] = None,
                    max_batch: int = 64, max_tokens_per_step: int = 8192, chunk_size: int = 512,
                    use_graphs: bool = True) -> "JiugeForCauslLM":
        """A model of a named configuration (``config.PRESETS``) with random weights from ``seed``.  Small ones are
        written as a model folder (config.json + model.safetensors, the ordinary loading path; the folder is removed
        afterwards); the large shapes are made on the device, where their checkpoint would be gigabytes on disk."""
        import shutil
        import tempfile
        from .config import PRESETS, MiniCPMConfig, config_class_for
        from .parts import model_manifest
        from .weights import DeviceRandomWeights, write_model_folder
        if preset not in PRESETS:
            raise ValueError(f"no configuration named {preset!r}; known: {', '.join(sorted(PRESETS))}")
        p = PRESETS[preset]
        page = page_size or p.page_size
        config = config_class_for(p.config).from_dict(p.config, max_tokens=max_tokens)
        spec = config.model_spec()
        small = sum(_numel(d.shape) for d in model_manifest(spec).values()) < (1 << 26)
        if small:
            folder = tempfile.mkdtemp(prefix=f"jiuge_{preset}_")
            try:
                write_model_folder(config, folder, seed=seed, std=p.std, norm_std=p.norm_std)
                return cls(folder, max_tokens=max_tokens, dtype=dtype, device_id=device_id, cache_tokens=cache_tokens,
                           page_size=page, num_pages=num_pages, max_batch=max_batch,
                           max_tokens_per_step=max_tokens_per_step, chunk_size=chunk_size, use_graphs=use_graphs)
            finally:
                shutil.rmtree(folder, ignore_errors=True)
        t0 = time.time()
        print("Loading model weights to device...")
        dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        dev = f"cuda:{device_id}"
        weights = DeviceRandomWeights(model_manifest(spec), seed=seed, compute_dtype=dt, device=dev, std=p.std,
                                      norm_std=p.norm_std, untied=not config.tie_word_embeddings)
        if num_pages is not None:
            cache_tokens = num_pages * page
        ctx = config.max_position_embeddings
        engine = Engine(spec, weights, dtype=dt, device=dev, cache_tokens=cache_tokens or max(ctx * min(max_batch, 4), 4096),
                        page_size=page, max_requests=max_batch, max_step_tokens=max_tokens_per_step, use_graphs=use_graphs)
        engine.config = config
        self = cls.from_engine(engine, max_batch, max_tokens_per_step, chunk_size)
        print(f"Time used: {time.time() - t0:.3f}s")
        return self

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
        logits = self.engine.step(self._entries(tasks), stage_next=True)
        params = [SamplingParams(t.temperature, t.topk, t.topp, getattr(t, "seed", self.sample_seed)) for t in tasks]
        return self.sampler.sample(logits, params, [t.pos + len(t.tokens) for t in tasks])

    def forward_batch(self, tasks: List[InferTask]) -> torch.Tensor:
        """Logits of every fed row, float32 on the device (the reference's ``forwardBatch``); the tensor is the
        caller's own: no later step writes into it."""
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
    """``jiuge.py --nvidia <model_dir> [n_device]`` as in scripts/jiuge.py:646-677, plus options; ``--random NAME``
    stands in for the model folder."""
    argv = list(sys.argv[1:] if argv is None else argv)
    usage = ("Usage: python -m infinicore_infer_b200.jiuge [--cpu | --nvidia | --cambricon | --ascend | --metax | "
             "--moore | --iluvatar] (<path/to/model_dir> [n_device] | --random NAME [--seed N]) "
             "[--dtype bfloat16|float32] [--prompt-ids 1,2,3 | --prompt TEXT | --prompt-len N | --prompt-lens N,N,..] "
             "[--max-steps N] [--temperature F] [--topk N] [--topp F] [--sample-seed N] [--max-tokens N] [--requests N] "
             "[--page-size N] [--num-pages N] [--max-batch N] [--max-tokens-per-step N] [--chunk-size N] [--device-id N]")
    if len(argv) < 2 or argv[0] not in _DEVICE_FLAGS:
        print(usage)
        return 1
    device = _DEVICE_FLAGS[argv[0]]
    if device != DeviceType.DEVICE_TYPE_NVIDIA:
        print(f"{argv[0]}: this engine is written for NVIDIA sm_100a only; use --nvidia")
        return 1
    from .config import PRESETS
    ap = argparse.ArgumentParser(prog="jiuge", usage=usage)
    ap.add_argument("model_dir", nargs="?", default=None)
    ap.add_argument("n_device", nargs="?", type=int, default=1)
    ap.add_argument("--random", default=None, choices=sorted(PRESETS), metavar="NAME",
                    help="instead of a model folder: a named configuration with random weights (" + ", ".join(sorted(PRESETS)) + ")")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights and of a random prompt")
    ap.add_argument("--dtype", default="bfloat16", choices=sorted(_DTYPES))
    ap.add_argument("--prompt", default=None, help="text (needs a tokenizer in the model folder)")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    ap.add_argument("--prompt-len", type=int, default=16, help="random prompt of this length if none is given")
    ap.add_argument("--prompt-lens", default=None, help="comma-separated lengths: one random prompt per request")
    ap.add_argument("--max-steps", "--max-new-tokens", dest="max_steps", type=int, default=500,
                    help="tokens to generate (scripts/jiuge.py:676 runs 500)")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--topk", type=int, default=1, help="1 (the reference's default) is greedy; 0 turns the limit off")
    ap.add_argument("--topp", type=float, default=1.0)
    ap.add_argument("--sample-seed", type=int, default=None, help="seed of the drawn tokens (default: --seed)")
    ap.add_argument("--max-tokens", type=int, default=None, help="context length override (the reference's max_tokens)")
    ap.add_argument("--requests", type=int, default=1, help="generate for this many requests at once, through the scheduler")
    ap.add_argument("--page-size", type=int, default=None, help="tokens per cache page (default 16; a named configuration's own)")
    ap.add_argument("--num-pages", type=int, default=None, help="pages of the pool that all requests share")
    ap.add_argument("--max-batch", type=int, default=64, help="most requests in one step")
    ap.add_argument("--max-tokens-per-step", type=int, default=8192, help="most tokens in one step")
    ap.add_argument("--chunk-size", type=int, default=512, help="most tokens of one prompt in one step")
    ap.add_argument("--device-id", type=int, default=0)
    args = ap.parse_args(argv[1:])
    if args.n_device != 1:
        print("n_device must be 1: this engine runs on one GPU")
        return 1
    if (args.model_dir is None) == (args.random is None):
        print("give a model folder or --random NAME (one of them)\n" + usage)
        return 1
    common = dict(max_tokens=args.max_tokens, dtype=args.dtype, device_id=args.device_id, num_pages=args.num_pages,
                  max_batch=args.max_batch, max_tokens_per_step=args.max_tokens_per_step, chunk_size=args.chunk_size)
    if args.random:
        model = JiugeForCauslLM.from_random(args.random, seed=args.seed, page_size=args.page_size, **common)
    else:
        model = JiugeForCauslLM(args.model_dir, device, args.n_device, page_size=args.page_size or 16, **common)
    vocab = model.engine.spec.vocab_size
    sample_seed = args.seed if args.sample_seed is None else args.sample_seed

    def random_prompt(n: int, k: int) -> List[int]:
        g = torch.Generator().manual_seed(args.seed + k)
        return torch.randint(0, vocab, (n,), generator=g).tolist()

    if args.prompt is not None:
        prompt = args.prompt
    elif args.prompt_ids:
        prompt = [int(t) for t in args.prompt_ids.split(",")]
    else:
        prompt = random_prompt(args.prompt_len, 0)
    if args.requests > 1 or args.prompt_lens:
        if args.prompt_lens:
            lens = [int(n) for n in args.prompt_lens.split(",")]
            prompts = [random_prompt(n, k) for k, n in enumerate(lens)]
        else:
            ids = model._encode(prompt) if isinstance(prompt, str) else prompt
            prompts = [ids] * args.requests
        t0 = time.time()
        outs = model.generate_batch(prompts, max_new_tokens=args.max_steps,
                                    temperature=0.0 if args.topk == 1 else args.temperature,
                                    topk=args.topk, topp=args.topp, seed=sample_seed)
        dt = time.time() - t0
        n = sum(len(o) for o in outs)
        for i, o in enumerate(outs):
            print(f"request {i}: {' '.join(str(t) for t in o)}")
        counters = model.generator.scheduler.counters
        print(f"{n} tokens for {len(prompts)} requests in {dt:.3f}s: {n / dt:.1f} tok/s; "
              f"{counters['steps']} steps, {counters['preemptions']} preemptions")
    else:
        model.generate(prompt, args.max_steps, topp_=args.topp, topk_=args.topk, temperature_=args.temperature,
                       seed=sample_seed)
    model.destroy_model_instance()
    return 0


if __name__ == "__main__":
    sys.exit(test())
