"""A plain, slow GPT-2 forward pass: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It is written from the formulas of
the reference engine (file:line cited at each function, paths within
mneha05/hetero-serve) and shares no code with ``hetero_serve_b200``: it takes a
raw ``config.json`` dictionary and a ``{name: tensor}`` dictionary, and computes
in float64 unless told otherwise.

``tests/golden/make_golden.py`` ran the reference's own CPU engine
(heteroserve/model/numpy_engine.py) once on a tiny random model; the outputs
committed beside it anchor this implementation (tests/test_plain.py).  The
options the reference does not have (``n_inner``, the erf GELU,
``scale_attn_by_inverse_layer_idx``, ``scale_attn_weights``) rest on the
formulas alone.
"""

from __future__ import annotations

import math

import torch

SQRT_2_OVER_PI = 0.7978845608028654     # heteroserve/model/numpy_engine.py:23


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------


def embed(wte, wpe, token_ids, positions):
    """x[t] = wte[ids[t]] + wpe[pos[t]]  (heteroserve/model/numpy_engine.py:80-81,
    heteroserve/model/torch_engine.py:89-90)."""
    return wte[token_ids] + wpe[positions]


def layer_norm(x, gamma, beta, eps):
    """mu = mean(x); xc = x - mu; var = mean(xc^2) (biased);
    y = xc / sqrt(var + eps) * g + b  (heteroserve/model/numpy_engine.py:26-30)."""
    mu = x.mean(dim=-1, keepdim=True)
    xc = x - mu
    var = (xc * xc).mean(dim=-1, keepdim=True)
    return xc / torch.sqrt(var + eps) * gamma + beta


def gelu_new(u):
    """0.5*u*(1 + tanh(sqrt(2/pi)*(u + 0.044715*u^3)))
    (heteroserve/model/numpy_engine.py:33-36; torch_engine.py:78 ``approximate="tanh"``)."""
    inner = SQRT_2_OVER_PI * (u + 0.044715 * u * u * u)
    return 0.5 * u * (1.0 + torch.tanh(inner))


def gelu_erf(u):
    """The exact GELU, 0.5*u*(1 + erf(u/sqrt(2))).  The reference has only the tanh
    form; this is the ``activation_function: "gelu"`` of GPT-2's configuration."""
    return 0.5 * u * (1.0 + torch.erf(u / math.sqrt(2.0)))


ACTIVATIONS = {"gelu_new": gelu_new, "gelu_pytorch_tanh": gelu_new, "gelu": gelu_erf}


def conv1d(x, weight, bias):
    """GPT-2's Conv1D: weight is [in, out]; y = x @ W + b
    (heteroserve/model/numpy_engine.py:123, torch_engine.py:122)."""
    return x @ weight + bias


def split_heads(t, n_head):
    """[T, H*D] -> [H, T, D]; head h is columns h*D..(h+1)*D
    (heteroserve/model/numpy_engine.py:60-64)."""
    T = t.shape[0]
    return t.reshape(T, n_head, -1).permute(1, 0, 2)


def softmax(x):
    """Max-subtracted softmax over the last axis (heteroserve/model/numpy_engine.py:39-42)."""
    m = x.max(dim=-1, keepdim=True).values
    e = torch.exp(x - m)
    return e / e.sum(dim=-1, keepdim=True)


def attention_scale(head_dim, layer_idx, scale_attn_weights=True, inverse_layer_idx=False):
    """1/sqrt(head_dim) (heteroserve/model/torch_engine.py:47), optionally divided by
    layer_idx + 1 (zero-based).  Formed in float64, rounded to 32-bit once: the
    kernels apply exactly this number."""
    s = 1.0 / math.sqrt(head_dim) if scale_attn_weights else 1.0
    if inverse_layer_idx:
        s = s / float(layer_idx + 1)
    return float(torch.tensor(s, dtype=torch.float64).to(torch.float32))


def causal_attention(q, k, v, scale, window=None):
    """scores = (q @ k^T) * scale; key j is visible to query i iff j <= i (and, with a
    window w, j > i - w); softmax; @ v; heads concatenated back to [T, H*D]
    (heteroserve/model/numpy_engine.py:111-145, torch_engine.py:112-139).
    q, k, v: [H, T, D]."""
    H, T, D = q.shape
    scores = (q @ k.transpose(1, 2)) * scale
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    blocked = j > i
    if window is not None:
        blocked = blocked | (j <= i - window)
    scores = scores.masked_fill(blocked.unsqueeze(0), float("-inf"))
    ctx = softmax(scores) @ v
    return ctx.permute(1, 0, 2).reshape(T, H * D)


def attention_block(h, w, prefix, n_head, scale):
    """qkv = h @ c_attn + b, split by columns into q | k | v, causal attention, c_proj
    (heteroserve/model/numpy_engine.py:122-146)."""
    E = h.shape[1]
    qkv = conv1d(h, w[prefix + "attn.c_attn.weight"], w[prefix + "attn.c_attn.bias"])
    q = split_heads(qkv[:, :E], n_head)
    k = split_heads(qkv[:, E:2 * E], n_head)
    v = split_heads(qkv[:, 2 * E:], n_head)
    ctx = causal_attention(q, k, v, scale)
    return conv1d(ctx, w[prefix + "attn.c_proj.weight"], w[prefix + "attn.c_proj.bias"])


def mlp_block(h, w, prefix, act):
    """act(h @ c_fc + b) @ c_proj + b  (heteroserve/model/numpy_engine.py:76-78)."""
    u = conv1d(h, w[prefix + "mlp.c_fc.weight"], w[prefix + "mlp.c_fc.bias"])
    return conv1d(act(u), w[prefix + "mlp.c_proj.weight"], w[prefix + "mlp.c_proj.bias"])


def lm_logits(x, w, eps):
    """ln_f then the tied head: LN_f(x) @ wte^T, no bias
    (heteroserve/model/numpy_engine.py:83-85, heteroserve/model/weights.py:40-43)."""
    h = layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["wte.weight"]
    return h @ head.T


# ---------------------------------------------------------------------------
# the whole model
# ---------------------------------------------------------------------------


def _strip(name):
    """Checkpoint prefixes the reference drops (heteroserve/model/weights.py:54-58)."""
    for p in ("transformer.", "model."):
        if name.startswith(p):
            return name[len(p):]
    return name


def prepare_weights(tensors, dtype=torch.float64, round_to=None):
    """Strip prefixes and convert.  ``round_to=torch.bfloat16`` first rounds the
    matrices and tables (tensors of two dimensions) to bfloat16, the precision the serving
    path stores them in, so that a comparison isolates the arithmetic."""
    out = {}
    for name, t in tensors.items():
        t = t.detach().cpu()
        if round_to is not None and t.dim() == 2 and t.dtype.is_floating_point:
            t = t.to(round_to)
        out[_strip(name)] = t.to(dtype) if t.dtype.is_floating_point else t
    return out


def forward(config, weights, token_ids, dtype=torch.float64, start_pos=0, rows=None):
    """Logits [T, vocab] of one whole sequence (positions start_pos..start_pos+T-1,
    nothing cached); with ``rows`` only the logits of these places, [len(rows), vocab]
    (the head is the costly part of a long sequence).  Pre-LayerNorm blocks on a residual
    stream, in the reference's order (heteroserve/model/numpy_engine.py:120-150):
        x = wte[ids] + wpe[pos]
        x = x + attn(ln_1(x));  x = x + mlp(ln_2(x))    for each layer
        logits = ln_f(x) @ wte^T
    """
    w = weights
    n_layer, n_head, E = config["n_layer"], config["n_head"], config["n_embd"]
    eps = config.get("layer_norm_epsilon", 1e-5)
    act = ACTIVATIONS[config.get("activation_function", "gelu_new")]
    n_pos = config.get("n_positions", config.get("n_ctx"))
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    T = ids.shape[0]
    if start_pos + T > n_pos:
        raise ValueError(f"{start_pos + T} positions exceed n_positions={n_pos}")
    pos = torch.arange(start_pos, start_pos + T)
    x = embed(w["wte.weight"], w["wpe.weight"], ids, pos).to(dtype)
    for i in range(n_layer):
        p = f"h.{i}."
        scale = attention_scale(E // n_head, i, config.get("scale_attn_weights", True),
                                config.get("scale_attn_by_inverse_layer_idx", False))
        h = layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps)
        x = x + attention_block(h, w, p, n_head, scale)
        h = layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps)
        x = x + mlp_block(h, w, p, act)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    return lm_logits(x, w, eps)


def greedy_generate(config, weights, prompt_ids, max_new_tokens, eos_token_id=None,
                    dtype=torch.float64):
    """Re-run the whole sequence for every new token and take the argmax (lowest index
    on ties), stopping after an end-of-sequence token or at the table's length
    (heteroserve/worker/worker.py:43-45, 714-715)."""
    ids = list(prompt_ids)
    out = []
    n_pos = config.get("n_positions", config.get("n_ctx"))
    for _ in range(max_new_tokens):
        if len(ids) > n_pos:
            break
        logits = forward(config, weights, ids, dtype)[-1]
        tok = int(torch.argmax(logits))
        out.append(tok)
        ids.append(tok)
        if eos_token_id is not None and tok == eos_token_id:
            break
        if len(ids) >= n_pos:
            break
    return out


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------

_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key, rounds=10):
    """Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
    counter: 4 words, key: 2 words → 4 words."""
    c = [int(x) & 0xFFFFFFFF for x in counter]
    k = [int(x) & 0xFFFFFFFF for x in key]
    for _ in range(rounds):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + _PHILOX_W0) & 0xFFFFFFFF, (k[1] + _PHILOX_W1) & 0xFFFFFFFF]
    return c


def uniform_for(seed, position):
    """The uniform number in [0, 1) that decides the token sampled at ``position`` (the
    index the new token will take in the sequence) of a request with ``seed``.  It
    depends on nothing else, so sampling does not depend on batching: the reference
    reseeds its generator with seed + n_kv for the same reason
    (heteroserve/worker/worker.py:647,694)."""
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    word = philox4x32([position & 0xFFFFFFFF, 0, 0, 0], [seed & 0xFFFFFFFF, seed >> 32])[0]
    return (word >> 8) * (1.0 / 16777216.0)


def sample_token(logits, temperature, top_k, u):
    """The reference's sampler (heteroserve/worker/worker.py:38-50) with the random draw
    made explicit: temperature <= 0 → argmax; else softmax(logits / temperature) in
    float64 over all tokens or, for 0 < top_k < V, over the top_k largest; the token is
    the first (in index order) whose cumulative probability exceeds ``u``."""
    logits = torch.as_tensor(logits, dtype=torch.float64)
    if temperature <= 0.0:
        return int(torch.argmax(logits))
    lg = logits / temperature
    V = lg.shape[0]
    keep = torch.ones(V, dtype=torch.bool)
    if top_k and 0 < top_k < V:
        # the k largest; ties at the threshold go to the lower indices
        order = sorted(range(V), key=lambda i: (-float(lg[i]), i))[:top_k]
        keep = torch.zeros(V, dtype=torch.bool)
        keep[order] = True
    m = lg[keep].max()
    e = torch.where(keep, torch.exp(lg - m), torch.zeros_like(lg))
    cdf = torch.cumsum(e, 0)
    target = u * float(cdf[-1])
    idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
    idx = min(idx, V - 1)
    while not keep[idx]:            # only reachable through rounding at the very end
        idx -= 1
    return idx
