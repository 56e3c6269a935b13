"""Plain, slow implementation of the GPT-2 style decoder: the oracle of the tests.

Whole sequences, no cache, one function per part, 64-bit by default, plain torch on the
CPU.  It shares no code with the engine.  Every function cites the lines of the
reference whose formula it restates.  ``tests/golden/make_golden.py`` compares it once
with the reference's own ``ReferenceGPT`` on a tiny random model and stores the logits.
"""

from __future__ import annotations

import math

import torch


def embed(tokens: torch.Tensor, w: dict, dtype=torch.float64) -> torch.Tensor:
    """x[t] = tok_emb[token_t] + pos_emb[t]        (src/minigpt_infer/model.py:183;
    positions are 0..T-1 as in src/minigpt_infer/reference.py:110-111)."""
    T = tokens.shape[0]
    if T > w["pos_emb.weight"].shape[0]:
        # src/minigpt_infer/model.py:177-182 / reference.py:109
        raise ValueError("sequence longer than the position table")
    return w["tok_emb.weight"].to(dtype)[tokens] + w["pos_emb.weight"].to(dtype)[:T]


def layer_norm(x: torch.Tensor, gain: torch.Tensor, shift: torch.Tensor | None,
               eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(biased var + eps) * gain + shift over the last axis
    (nn.LayerNorm as used at src/minigpt_infer/model.py:107-109, 127)."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    y = (x - mean) / torch.sqrt(var + eps) * gain.to(x.dtype)
    return y + shift.to(x.dtype) if shift is not None else y


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """x @ W^T + b with W stored [out, in]   (nn.Linear, src/minigpt_infer/model.py:43-44)."""
    y = x @ weight.to(x.dtype).T
    return y + bias.to(x.dtype) if bias is not None else y


def gelu_tanh(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))
    (F.gelu(approximate="tanh"), src/minigpt_infer/model.py:101)."""
    return 0.5 * u * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (u + 0.044715 * u ** 3)))


def causal_attention(x: torch.Tensor, w: dict, prefix: str, n_head: int,
                     window: int | None = None, n_kv_head: int | None = None,
                     scale: float | None = None) -> torch.Tensor:
    """q,k,v = split(x W_qkv^T + b) in that order, head h = columns [hD,(h+1)D);
    softmax(q k^T / sqrt(D) + causal mask) v; heads side by side; output projection
    (src/minigpt_infer/model.py:48-53, 87-90; reference.py:38-50).  ``window`` and
    ``n_kv_head`` are not used by this architecture; the engine's parts take them."""
    T, C = x.shape
    n_kv = n_kv_head or n_head
    qkv = linear(x, w[prefix + "qkv.weight"], w.get(prefix + "qkv.bias"))
    D = qkv.shape[1] // (n_head + 2 * n_kv)
    q = qkv[:, : n_head * D].reshape(T, n_head, D)
    k = qkv[:, n_head * D: (n_head + n_kv) * D].reshape(T, n_kv, D)
    v = qkv[:, (n_head + n_kv) * D:].reshape(T, n_kv, D)
    s = (1.0 / math.sqrt(D)) if scale is None else scale
    out = torch.zeros(T, n_head, D, dtype=x.dtype)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    for h in range(n_head):
        kh = h // (n_head // n_kv)
        scores = (q[:, h] @ k[:, kh].T) * s
        scores = scores.masked_fill(~allowed, float("-inf"))
        out[:, h] = torch.softmax(scores, dim=-1) @ v[:, kh]
    return linear(out.reshape(T, n_head * D), w[prefix + "proj.weight"], w.get(prefix + "proj.bias"))


def mlp(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """proj(gelu_tanh(fc(x)))                      (src/minigpt_infer/model.py:100-101)."""
    h = gelu_tanh(linear(x, w[prefix + "fc.weight"], w.get(prefix + "fc.bias")))
    return linear(h, w[prefix + "proj.weight"], w.get(prefix + "proj.bias"))


def block(x: torch.Tensor, w: dict, prefix: str, n_head: int, eps: float) -> torch.Tensor:
    """x = x + attn(ln1(x)); x = x + mlp(ln2(x))   (src/minigpt_infer/model.py:112-115)."""
    x = x + causal_attention(layer_norm(x, w[prefix + "ln1.weight"], w.get(prefix + "ln1.bias"),
                                        eps), w, prefix + "attn.", n_head)
    x = x + mlp(layer_norm(x, w[prefix + "ln2.weight"], w.get(prefix + "ln2.bias"), eps),
                w, prefix + "mlp.")
    return x


def forward_logits(tokens, w: dict, n_layer: int, n_head: int, eps: float = 1e-5,
                   dtype=torch.float64, rows=None) -> torch.Tensor:
    """Logits at every position of one whole sequence: embed, blocks in order, final
    LayerNorm, tied head without bias (src/minigpt_infer/reference.py:105-114,
    src/minigpt_infer/model.py:128-130, 183-187).  ``rows``: only these positions meet the
    head (the whole sequence still runs through the blocks); with a vocabulary of tens of
    thousands the head is most of the work."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = embed(tokens, w, dtype)
    for i in range(n_layer):
        x = block(x, w, f"blocks.{i}.", n_head, eps)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    x = layer_norm(x, w["ln_f.weight"], w.get("ln_f.bias"), eps)
    return x @ w["tok_emb.weight"].to(dtype).T


def greedy_generate(tokens, w: dict, n_layer: int, n_head: int, eps: float,
                    max_new_tokens: int) -> list[int]:
    """Full re-forward each step, argmax of the last position
    (src/minigpt_infer/reference.py:149-175)."""
    seq = list(tokens)
    for _ in range(max_new_tokens):
        seq.append(int(forward_logits(seq, w, n_layer, n_head, eps)[-1].argmax()))
    return seq[len(tokens):]


# ---- sampling ----------------------------------------------------------------------------
def top_k_filter(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Keep values >= the k-th largest (ties pass) (src/minigpt_infer/sampling.py:39-52)."""
    k = max(1, min(int(k), logits.shape[-1]))
    thr = torch.sort(logits, descending=True).values[..., k - 1]
    return logits.masked_fill(logits < thr[..., None], float("-inf"))


def top_p_filter(logits: torch.Tensor, p: float) -> torch.Tensor:
    """Sorted descending, drop a token if the mass strictly before it exceeds p; the first
    is always kept (src/minigpt_infer/sampling.py:55-76)."""
    vals, idx = torch.sort(logits, descending=True)
    probs = torch.softmax(vals, dim=-1)
    before = probs.cumsum(-1) - probs
    remove = before > p
    remove[..., 0] = False
    vals = vals.masked_fill(remove, float("-inf"))
    return torch.full_like(logits, float("-inf")).scatter(-1, idx, vals)


def sampling_distribution(logits: torch.Tensor, temperature: float, top_k=None,
                          top_p=None) -> torch.Tensor:
    """The distribution the sampler draws from: logits / max(T, 1e-6) -> top-k -> top-p ->
    softmax (src/minigpt_infer/sampling.py:116-131)."""
    x = logits.to(torch.float64) / max(float(temperature), 1e-6)
    if top_k is not None:
        x = top_k_filter(x, top_k)
    if top_p is not None:
        x = top_p_filter(x, top_p)
    return torch.softmax(x, dim=-1)
