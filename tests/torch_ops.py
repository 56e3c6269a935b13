"""A kernel set written with plain torch, for tests that run the engine's step function,
cache and parts without a GPU.  It is a test double: the product path has no such set and
refuses to run without its CUDA extension.  It follows the same calling conventions and
cache layout as the CUDA kernel set, and shares nothing with ``plain_gpt``.
"""

from __future__ import annotations

import math

import torch


class TorchOps:
    name = "torch-test-double"

    def embed(self, token_ids, positions, tok_emb, pos_table):
        x = tok_emb.float()[token_ids.long()]
        if pos_table is not None:
            x = x + pos_table.float()[positions.long()]
        return x

    def layernorm(self, x32, gain, shift, eps, out_dtype):
        mean = x32.mean(-1, keepdim=True)
        var = ((x32 - mean) ** 2).mean(-1, keepdim=True)
        y = (x32 - mean) * torch.rsqrt(var + eps) * gain
        if shift is not None:
            y = y + shift
        return y.to(out_dtype)

    def linear(self, x, weight, bias, activation, out_dtype):
        y = x.float() @ weight.float().T
        if bias is not None:
            y = y + bias
        if activation == "gelu_tanh":
            y = 0.5 * y * (1 + torch.tanh(math.sqrt(2 / math.pi) * (y + 0.044715 * y ** 3)))
        elif activation != "none":
            raise ValueError(activation)
        return y.to(out_dtype)

    def linear_residual(self, x, weight, bias, residual32):
        y = x.float() @ weight.float().T
        if bias is not None:
            y = y + bias
        residual32 += y

    def kv_store(self, qkv, n_head, n_kv_head, head_dim, cache, slot_mapping):
        N = qkv.shape[0]
        k = qkv[:, n_head * head_dim: (n_head + n_kv_head) * head_dim].reshape(N, n_kv_head, head_dim)
        v = qkv[:, (n_head + n_kv_head) * head_dim:].reshape(N, n_kv_head, head_dim)
        slots = slot_mapping.long()
        page, off = slots // cache.page_tokens, slots % cache.page_tokens
        cache.k_pages[page, :, off] = k.to(cache.k_pages.dtype)
        cache.v_pages[page, :, off] = v.to(cache.v_pages.dtype)

    def paged_attention(self, qkv, n_head, n_kv_head, head_dim, scale, cache, ctx):
        N = qkv.shape[0]
        q = qkv[:, : n_head * head_dim].reshape(N, n_head, head_dim).float()
        out = torch.zeros(N, n_head, head_dim)
        table = ctx.block_tables[cache.group].long()
        pt = cache.page_tokens
        for i in range(N):
            r = int(ctx.token_request[i])
            p = int(ctx.positions[i])
            lo = 0 if cache.window is None else max(0, p - cache.window + 1)
            keys = torch.arange(lo, p + 1)
            pages = table[r, keys // pt]
            assert (pages >= 0).all(), "attention reads a page that is not there"
            k = cache.k_pages[pages, :, keys % pt].float()      # [keys, Hkv, D]
            v = cache.v_pages[pages, :, keys % pt].float()
            for h in range(n_head):
                kh = h // (n_head // n_kv_head)
                s = (k[:, kh] @ q[i, h]) * scale
                out[i, h] = torch.softmax(s, dim=0) @ v[:, kh]
        return out.reshape(N, n_head * head_dim).to(qkv.dtype)

    def gather_rows(self, x32, rows):
        return x32[rows.long()]

    def logits(self, y, tok_emb):
        return y.float() @ tok_emb.float().T

    def argmax(self, logits, vocab_limit=None, out=None):
        v = logits if vocab_limit is None else logits[:, :vocab_limit]
        ids = v.argmax(-1).to(torch.int32)
        if out is None:
            return ids
        out.copy_(ids)
        return out
