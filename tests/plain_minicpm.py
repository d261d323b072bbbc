"""A plain, slow implementation of the MiniCPM/FM9G decoder for the tests.

Whole sequences, no cache, one function for each part, plain torch on the CPU; it shares no
code with the engine.  It RESTS ON THE REFERENCE'S FORMULAS, not on running the reference:
InfiniCore-Infer's model code (src/models/jiuge/*.cpp) calls the external libraries
infiniop / infinirt / infiniccl, which are absent here, so it can be neither compiled nor
imported on this machine.  Each function cites the file:line of the reference it restates.

Weights are taken by their checkpoint names, unpermuted.  The reference's loader permutes
the rows of the query and key matrices inside each head so that its rotary operator can
turn adjacent pairs (scripts/jiuge.py:217-227); turning pair (j, j + dh/2) of the unpermuted
rows with the same angle is the same function, and that is what ``plain_rope`` does.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def plain_scales(cfg: dict):
    """(embedding scale, residual scale, logit scale).  scripts/jiuge.py:97-114: the scales
    apply when model_type is fm9g or minicpm and the three keys are present; the logit scale
    is hidden_size // dim_model_base and MULTIPLIES (it is folded into the final norm's
    weight, scripts/jiuge.py:198-201)."""
    if (cfg.get("model_type") in ("fm9g", "minicpm") and "scale_emb" in cfg
            and "scale_depth" in cfg and "dim_model_base" in cfg):
        return (float(cfg["scale_emb"]),
                float(cfg["scale_depth"]) / math.sqrt(cfg["num_hidden_layers"]),
                float(cfg["hidden_size"] // cfg["dim_model_base"]))
    return 1.0, 1.0, 1.0


def plain_embedding(tokens: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """x[i] = (E * scale_emb)[tokens[i]].  src/models/jiuge/jiuge.cpp:164-168, scripts/jiuge.py:194-197."""
    return table[tokens] * scale


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * w / sqrt(mean(x^2) + eps) over the last dimension.  src/models/jiuge/jiuge.cpp:198."""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def plain_rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate heads ``x [T, H, dh]``: pair (j, j + dh/2) by the angle pos / theta^(j/(dh/2)).
    Tables: src/models/jiuge/jiuge_weight.hpp:134-186; pairing: scripts/jiuge.py:217-227;
    applied to query and key heads at src/models/jiuge/jiuge.cpp:202-203."""
    dh = x.shape[-1]
    half = dh // 2
    j = torch.arange(half, dtype=torch.float64)
    angle = positions.to(torch.float64)[:, None] / (float(theta) ** (j / half))[None, :]
    cos = angle.cos().to(x.dtype)[:, None, :]
    sin = angle.sin().to(x.dtype)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    window: Optional[int] = None) -> torch.Tensor:
    """Causal softmax attention of a whole sequence.  q [T, nh, dh]; k, v [T, nkvh, dh].
    Query head h uses key/value head h // (nh / nkvh); row i sees columns j <= i (and
    j > i - window if a window is given).  src/models/jiuge/jiuge.cpp:210-230 (scale 1/sqrt(dh)
    at :223, causal softmax at :225-226)."""
    T, nh, dh = q.shape
    g = nh // k.shape[1]
    out = torch.empty_like(q)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    mask = j <= i
    if window:
        mask = mask & (j > i - window)
    for h in range(nh):
        s = (q[:, h, :] @ k[:, h // g, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h // g, :]
    return out


def plain_swiglu_ffn(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)), silu(z) = z * sigmoid(z).  src/models/jiuge/jiuge.cpp:247-249."""
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def plain_attention_layer(h, w: Dict[str, torch.Tensor], prefix: str, positions, nh, nkvh, dh, theta,
                          window=None, kv_override=None):
    """QKV products, rope, attention, output product of one layer.  src/models/jiuge/jiuge.cpp:200-236.
    Returns (output, (k, v)) so that a layer that reads another layer's cache can be expressed."""
    T = h.shape[0]
    q = (h @ w[prefix + "q_proj.weight"].T)
    if prefix + "q_proj.bias" in w:
        q = q + w[prefix + "q_proj.bias"]
    q = plain_rope(q.view(T, nh, dh), positions, theta)
    if kv_override is None:
        k = h @ w[prefix + "k_proj.weight"].T
        v = h @ w[prefix + "v_proj.weight"].T
        if prefix + "k_proj.bias" in w:
            k = k + w[prefix + "k_proj.bias"]
            v = v + w[prefix + "v_proj.bias"]
        k = plain_rope(k.view(T, nkvh, dh), positions, theta)
        v = v.view(T, nkvh, dh)
    else:
        k, v = kv_override
    o = plain_attention(q, k, v, 1.0 / math.sqrt(dh), window)
    return o.reshape(T, nh * dh) @ w[prefix + "o_proj.weight"].T, (k, v)


def plain_forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
                  dtype: torch.dtype = torch.float64, windows: Optional[Sequence[Optional[int]]] = None,
                  order: Optional[Sequence[tuple]] = None, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence from position 0.  The step of the reference,
    src/models/jiuge/jiuge.cpp:114-298, for a single request with req_pos = 0.

    ``windows[i]``: attention window of layer i (None: full).  ``order``: run entries
    ``(layer, cache, writes_cache)``; the default runs every layer once with its own cache.
    ``rows``: compute the logits of these positions only (the final norm and the output product look at single
    rows, src/models/jiuge/jiuge.cpp:269-278); the result is then [len(rows), vocab].
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    L, d, nh = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"]
    nkvh = cfg.get("num_key_value_heads") or nh
    dh = cfg.get("head_dim") or d // nh
    theta = cfg.get("rope_theta", 100000.0)            # scripts/jiuge.py:133
    eps = cfg["rms_norm_eps"]
    scale_emb, scale_res, scale_logit = plain_scales(cfg)
    if "logit_scale" in cfg:
        scale_logit = float(cfg["logit_scale"])
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(tok))
    x = plain_embedding(tok, w["model.embed_tokens.weight"], scale_emb)
    order = order or [(i, i, True) for i in range(L)]
    caches = {}
    for layer, cache, writes in order:
        p = f"model.layers.{layer}."
        h = plain_rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        a, kv = plain_attention_layer(h, w, p + "self_attn.", positions, nh, nkvh, dh, theta,
                                      windows[layer] if windows else None,
                                      None if writes else caches[cache])
        if writes:
            caches[cache] = kv
        x = x + scale_res * a                                                    # jiuge.cpp:236, jiuge.py:297
        h = plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)     # jiuge.cpp:246
        x = x + scale_res * plain_swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                             w[p + "mlp.down_proj.weight"])      # jiuge.cpp:247-249, jiuge.py:348
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    h = plain_rmsnorm(x, w["model.norm.weight"], eps) * scale_logit             # jiuge.cpp:262, jiuge.py:198-201
    out = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]   # jiuge.py:182-191
    return h @ out.T                                                             # jiuge.cpp:264


def plain_greedy(cfg: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int], steps: int,
                 dtype: torch.dtype = torch.float64) -> List[int]:
    """Greedy continuation: the whole sequence is recomputed for every new token."""
    seq = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(plain_forward(cfg, weights, seq, dtype)[-1].argmax())
        out.append(nxt)
        seq.append(nxt)
    return out


def plain_sample(logits: torch.Tensor, temperature: float, topk: int, topp: float, u: float) -> int:
    """The engine's sampling rule, restated: greedy when temperature is 0 or topk is 1
    (include/infinicore_infer/models/jiuge.h:85-87); else candidates are the largest logits
    until topk of them or a share topp of the mass is reached (ties with the last one
    included), and the token is the first candidate in vocabulary order whose running mass
    exceeds u times the candidates' mass.  A token's mass is exp((logit - max) / temperature)
    counted in units of 2^-32, rounded down: a token less likely than that is never drawn."""
    logits = logits.to(torch.float64)
    V = logits.numel()
    if temperature <= 0 or topk == 1:
        return int(torch.argmax(logits))       # first maximal index
    z = logits / temperature
    w = torch.floor(torch.exp(z - z.max()) * 4294967296.0)
    total = w.sum()
    order = torch.argsort(z, descending=True, stable=True)
    kk = topk if 1 < topk < V else V
    limit = total * min(max(topp, 0.0), 1.0) if topp < 1 else total
    cnt, mass, tau = 0, 0.0, None
    zs = z[order]
    ws = w[order]
    i = 0
    while i < V:
        jx = i
        while jx < V and zs[jx] == zs[i]:
            jx += 1
        tau = zs[i]
        if cnt + (jx - i) >= kk or mass + float(ws[i:jx].sum()) >= float(limit):
            break
        cnt += jx - i
        mass += float(ws[i:jx].sum())
        i = jx
    cand = z >= tau
    cw = torch.where(cand, w, torch.zeros_like(w))
    target = torch.floor(u * cw.sum())
    cum = torch.cumsum(cw, 0)
    idx = torch.nonzero((cum > target) & cand)
    return int(idx[0]) if len(idx) else int(torch.nonzero(cand)[-1])
