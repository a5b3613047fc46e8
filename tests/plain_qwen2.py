"""Plain, slow Qwen2 dense decoder: the oracle every engine test compares against.

Whole sequences, no cache, no batching, one function per part, float32 unless a
caller passes other tensors.  It shares no code with ``distie_b200``: weights come
in as a plain ``dict`` of tensors keyed by checkpoint names and the sizes come in
as a plain ``dict`` holding the keys of ``config.json``.

Every function is written from the formulas of the reference project
(stanzixinwan/distie); the citation in each docstring is ``path:line`` inside
that project.  ``tests/golden/make_golden.py`` compared this file once with the
reference's own ``Qwen2CausalLM`` on the CPU and committed the small outputs.
"""

from __future__ import annotations

import math

import torch


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather ``h[t] = E[ids[t]]`` (worker/src/inference/qwen2/model.py:297,309)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Variance in float32, weight applied after the cast back.

    worker/src/inference/qwen2/model.py:85-90
    """
    dtype = x.dtype
    x32 = x.float()
    variance = (x32 * x32).mean(dim=-1, keepdim=True)
    return weight * (x32 * torch.rsqrt(variance + eps)).to(dtype)


def rope_inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
    """``inv_freq[j] = 1 / theta**(2j/d)`` (worker/src/inference/qwen2/model.py:98)."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    """cos/sin of ``cat(f, f)`` with ``f = pos * inv_freq``, evaluated in float32.

    worker/src/inference/qwen2/model.py:101-105
    """
    freqs = positions.float()[:, None] * rope_inverse_frequencies(head_dim, theta).to(positions.device)[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``cat(-x[d/2:], x[:d/2])``: pairs are (j, j + d/2) (model.py:115-117)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin`` for x ``[T, heads, d]`` (model.py:108-112)."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def visible_mask(num_tokens: int, window: int | None = None, device=None) -> torch.Tensor:
    """True where query ``i`` may see key ``j``: ``j <= i`` (model.py:128-135).

    ``window`` (not in the reference, which rejects windowed layers at
    model.py:58-60) additionally hides keys with ``i - j >= window``; toy layers of
    the tests use it.
    """
    i = torch.arange(num_tokens, device=device)[:, None]
    j = torch.arange(num_tokens, device=device)[None, :]
    mask = j <= i
    if window is not None:
        mask &= (i - j) < window
    return mask


def attention_mix(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window: int | None = None,
    scale: float | None = None,
) -> torch.Tensor:
    """Causal grouped-query attention of one sequence.

    q ``[T, nq, d]``, k and v ``[T, nkv, d]``; q head ``h`` uses kv head
    ``h // (nq // nkv)`` (model.py:120-125).  Scores are scaled by ``d**-0.5`` after
    the product, masked, soft-maxed in float32 and cast back (model.py:157-160).
    """
    num_tokens, nq, d = q.shape
    nkv = k.shape[1]
    rep = nq // nkv
    scale = d**-0.5 if scale is None else scale
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kk) * scale
    mask = visible_mask(num_tokens, window, q.device)
    scores = scores.masked_fill(~mask[None], torch.finfo(scores.dtype).min)
    weights = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.einsum("hts,shd->thd", weights, vv)


def attention_layer(
    x: torch.Tensor,
    w: dict,
    prefix: str,
    positions: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    theta: float,
    window: int | None = None,
    kv_from: tuple[torch.Tensor, torch.Tensor] | None = None,
):
    """q/k/v projections with bias, RoPE on q and k, mix, output projection without bias.

    worker/src/inference/qwen2/model.py:214-225.  Returns the output and the
    rotated (k, v) so that a toy layer order can let a later layer read them.
    """
    num_tokens = x.shape[0]
    q = torch.nn.functional.linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias"))
    k = torch.nn.functional.linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias"))
    v = torch.nn.functional.linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias"))
    q = q.view(num_tokens, num_heads, head_dim)
    k = k.view(num_tokens, num_kv_heads, head_dim)
    v = v.view(num_tokens, num_kv_heads, head_dim)
    cos, sin = rope_tables(positions, head_dim, theta)
    cos, sin = cos.to(x.dtype), sin.to(x.dtype)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    if kv_from is not None:
        k, v = kv_from
    mixed = attention_mix(q, k, v, window)
    out = torch.nn.functional.linear(mixed.reshape(num_tokens, num_heads * head_dim), w[prefix + "o_proj.weight"])
    return out, (k, v)


def swiglu_mlp(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))``, no biases (model.py:228-236)."""
    gate = torch.nn.functional.linear(x, w[prefix + "gate_proj.weight"])
    up = torch.nn.functional.linear(x, w[prefix + "up_proj.weight"])
    return torch.nn.functional.linear(torch.nn.functional.silu(gate) * up, w[prefix + "down_proj.weight"])


def decoder_layer(h, w, layer, positions, cfg, window=None, kv_from=None):
    """Pre-norm block with two residual sums (model.py:247-249)."""
    p = f"model.layers.{layer}."
    attn, kv = attention_layer(
        rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"]),
        w,
        p + "self_attn.",
        positions,
        cfg["num_attention_heads"],
        cfg["num_key_value_heads"],
        head_dim_of(cfg),
        rope_theta_of(cfg),
        window,
        kv_from,
    )
    h = h + attn
    h = h + swiglu_mlp(rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), w, p + "mlp.")
    return h, kv


def head_dim_of(cfg: dict) -> int:
    """Explicit ``head_dim`` or ``hidden_size // num_attention_heads`` (model.py:47-48)."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def rope_theta_of(cfg: dict) -> float:
    """``rope_parameters.rope_theta`` wins over ``rope_theta`` (model.py:413-419)."""
    params = cfg.get("rope_parameters") or {}
    if "rope_theta" in params:
        return float(params["rope_theta"])
    return float(cfg["rope_theta"])


def output_head(h: torch.Tensor, w: dict, cfg: dict) -> torch.Tensor:
    """Final norm, then the head; a tied head is the embedding table (model.py:299-303,314)."""
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return torch.nn.functional.linear(rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]), head)


def forward_logits(ids, w: dict, cfg: dict, order=None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence (model.py:305-314).

    ``order`` is a list of ``(layer, window, reads_kv_of)`` for toy arrangements;
    the architecture itself runs every layer once, in order, with full attention.
    """
    device = w["model.embed_tokens.weight"].device  # tensors on another device than the CPU: everything runs there
    ids = torch.as_tensor(ids, dtype=torch.long, device=device)
    positions = torch.arange(ids.shape[0], device=device)
    h = embedding(ids, w["model.embed_tokens.weight"])
    if order is None:
        order = [(i, None, None) for i in range(cfg["num_hidden_layers"])]
    kvs: dict[int, tuple] = {}
    for call, (layer, window, reads) in enumerate(order):
        h, kv = decoder_layer(h, w, layer, positions, cfg, window, kvs[reads] if reads is not None else None)
        kvs[call] = kv
    return output_head(h, w, cfg).float()


def greedy_generate(prompt, w: dict, cfg: dict, max_new_tokens: int, eos_id: int | None = None) -> list[int]:
    """Recompute the whole sequence for every new token; argmax (model_runner.py:124-125)."""
    ids = list(prompt)
    out: list[int] = []
    for _ in range(max_new_tokens):
        token = int(forward_logits(ids, w, cfg)[-1].argmax())
        out.append(token)
        ids.append(token)
        if eos_id is not None and token == eos_id:
            break
    return out


def temperature_probabilities(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """``softmax(logits / temperature)`` in float32 (model_runner.py:126-128)."""
    return torch.softmax(logits.float() / temperature, dim=-1)


def random_weights(cfg: dict, seed: int, std: float = 0.02, norm_noise: float = 0.0, dtype=torch.float32) -> dict:
    """Checkpoint-named random tensors for tests (names: model.py:386-400)."""
    g = torch.Generator().manual_seed(seed)
    hidden, inter, vocab = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)

    def mat(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def norm():
        return (torch.ones(hidden) + torch.randn(hidden, generator=g) * norm_noise).to(dtype)

    w = {"model.embed_tokens.weight": mat(vocab, hidden)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = mat(nq * d, hidden)
        w[p + "self_attn.q_proj.bias"] = mat(nq * d)
        w[p + "self_attn.k_proj.weight"] = mat(nkv * d, hidden)
        w[p + "self_attn.k_proj.bias"] = mat(nkv * d)
        w[p + "self_attn.v_proj.weight"] = mat(nkv * d, hidden)
        w[p + "self_attn.v_proj.bias"] = mat(nkv * d)
        w[p + "self_attn.o_proj.weight"] = mat(hidden, nq * d)
        w[p + "mlp.gate_proj.weight"] = mat(inter, hidden)
        w[p + "mlp.up_proj.weight"] = mat(inter, hidden)
        w[p + "mlp.down_proj.weight"] = mat(hidden, inter)
        w[p + "input_layernorm.weight"] = norm()
        w[p + "post_attention_layernorm.weight"] = norm()
    w["model.norm.weight"] = norm()
    if not cfg.get("tie_word_embeddings", False):
        w["lm_head.weight"] = mat(vocab, hidden)
    return w


def logit_scale(logits: torch.Tensor) -> float:
    """The number tolerances are relative to: the largest logit magnitude, at least 1."""
    return max(1.0, float(logits.abs().max()))


__all__ = [name for name in dir() if not name.startswith("_") and name not in {"math", "torch", "annotations"}]
