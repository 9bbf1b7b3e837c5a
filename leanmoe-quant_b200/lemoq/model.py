"""A transformers-free OLMoE module tree with the attribute names the lemoq op API patches.

The reference monkey-patches a Hugging Face ``OlmoeForCausalLM`` (transformers 4.57.6).  That
version is not what current images ship, so the host side carries its own minimal restatement of
the same module layout: ``model.model.layers[i].{input_layernorm, self_attn, post_attention_layernorm,
mlp}``, ``self_attn.{q,k,v,o}_proj`` + ``q_norm/k_norm`` on the full projection width,
``mlp.gate`` + ``mlp.experts[j].{gate,up,down}_proj``, ``model.norm``, untied ``lm_head`` and a
``StaticCache`` with ``layers[i].keys/values`` of shape ``(1, heads, max_len, head_dim)``.
``replace_rms_norms``, ``replace_moe_blocks``, ``quantize_model``, ``replace_attention_cores`` and
``install_packed_qkv`` all work on it.  The plain forwards here are the eager (prefill) path; the
decode hot path is the CUDA kernels.
"""

from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class OlmoeConfig:
    vocab_size: int = 50304
    hidden_size: int = 2048
    intermediate_size: int = 1024
    num_hidden_layers: int = 16
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    num_experts: int = 64
    num_experts_per_tok: int = 8
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    norm_topk_prob: bool = False
    clip_qkv: float | None = None
    initializer_range: float = 0.02
    model_type: str = "olmoe"
    output_attentions: bool = False

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


class OlmoeRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states: Any) -> Any:
        dt = hidden_states.dtype
        h = hidden_states.to(torch.float32)
        h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return self.weight * h.to(dt)


class OlmoeRotaryEmbedding(nn.Module):
    """cos/sin ``(B, L, D)`` in the dtype of ``x``.  The tables are evaluated on the host (CPU
    libm) and cached per device, so every device sees the same fp16 bits."""

    def __init__(self, config: OlmoeConfig) -> None:
        super().__init__()
        self.head_dim = config.head_dim
        self.theta = float(config.rope_theta)
        self._tables: dict[tuple, tuple[Any, Any]] = {}

    def tables(self, max_len: int, dtype: Any, device: Any) -> tuple[Any, Any]:
        key = (int(max_len), dtype, str(device))
        if key not in self._tables:
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.int64).float() / self.head_dim))
            freqs = torch.arange(max_len, dtype=torch.float32)[:, None] * inv_freq[None, :]
            emb = torch.cat((freqs, freqs), dim=-1)
            self._tables[key] = (emb.cos().to(dtype).to(device).contiguous(), emb.sin().to(dtype).to(device).contiguous())
        return self._tables[key]

    def forward(self, x: Any, position_ids: Any, max_len: int | None = None) -> tuple[Any, Any]:
        n = int(max_len) if max_len is not None else int(position_ids.max().item()) + 1
        cos, sin = self.tables(n, x.dtype, x.device)
        return cos[position_ids], sin[position_ids]


class OlmoeMLP(nn.Module):
    def __init__(self, config: OlmoeConfig) -> None:
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)
        self.act_fn = F.silu

    def forward(self, x: Any) -> Any:
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class OlmoeSparseMoeBlock(nn.Module):
    def __init__(self, config: OlmoeConfig) -> None:
        super().__init__()
        self.num_experts = config.num_experts
        self.top_k = config.num_experts_per_tok
        self.norm_topk_prob = config.norm_topk_prob
        self.act_fn = F.silu
        self.gate = nn.Linear(config.hidden_size, self.num_experts, bias=False)
        self.experts = nn.ModuleList([OlmoeMLP(config) for _ in range(self.num_experts)])

    def forward(self, hidden_states: Any) -> tuple[Any, Any]:
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        logits = self.gate(x)
        weights = F.softmax(logits, dim=1, dtype=torch.float)
        top_w, top_i = torch.topk(weights, self.top_k, dim=-1)
        if self.norm_topk_prob:
            top_w = top_w / top_w.sum(dim=-1, keepdim=True)
        top_w = top_w.to(x.dtype)
        out = torch.zeros_like(x)
        for e in range(self.num_experts):
            tok, slot = (top_i == e).nonzero(as_tuple=True)
            if tok.numel():
                out.index_add_(0, tok, self.experts[e](x[tok]) * top_w[tok, slot].unsqueeze(-1))
        return out.reshape(shape), logits


def _rotate_half(x: Any) -> Any:
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class OlmoeAttention(nn.Module):
    def __init__(self, config: OlmoeConfig, layer_idx: int) -> None:
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = config.head_dim
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        kv = self.num_key_value_heads * self.head_dim
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(self.hidden_size, kv, bias=False)
        self.v_proj = nn.Linear(self.hidden_size, kv, bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=False)
        self.q_norm = OlmoeRMSNorm(self.num_heads * self.head_dim, eps=config.rms_norm_eps)
        self.k_norm = OlmoeRMSNorm(kv, eps=config.rms_norm_eps)

    def forward(self, hidden_states: Any, attention_mask: Any = None, position_ids: Any = None,
                past_key_values: Any = None, output_attentions: bool = False, use_cache: bool = False,
                cache_position: Any = None, position_embeddings: Any = None, **kwargs: Any) -> tuple[Any, Any]:
        """Eager attention (prefill and reference arm): additive mask, fp32 softmax."""
        bsz, q_len, _ = hidden_states.shape
        q = self.q_norm(self.q_proj(hidden_states))
        k = self.k_norm(self.k_proj(hidden_states))
        v = self.v_proj(hidden_states)
        if self.config.clip_qkv is not None:
            c = self.config.clip_qkv
            q, k, v = q.clamp(-c, c), k.clamp(-c, c), v.clamp(-c, c)
        q = q.view(bsz, q_len, self.num_heads, self.head_dim).transpose(1, 2)
        k = k.view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = v.view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        cos, sin = position_embeddings
        cos_u, sin_u = cos.unsqueeze(1), sin.unsqueeze(1)
        q = (q * cos_u) + (_rotate_half(q) * sin_u)
        k = (k * cos_u) + (_rotate_half(k) * sin_u)
        if past_key_values is not None:
            k, v = past_key_values.update(k, v, self.layer_idx, {"sin": sin, "cos": cos, "cache_position": cache_position})
        if self.num_key_value_groups != 1:
            k = k.repeat_interleave(self.num_key_value_groups, dim=1)
            v = v.repeat_interleave(self.num_key_value_groups, dim=1)
        scores = torch.matmul(q, k.transpose(2, 3)) * (self.head_dim ** -0.5)
        if attention_mask is not None:
            scores = scores + attention_mask[:, :, :, : k.shape[-2]]
        w = F.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
        out = torch.matmul(w, v).transpose(1, 2).contiguous().reshape(bsz, q_len, self.hidden_size)
        return self.o_proj(out), (w if output_attentions else None)


class OlmoeDecoderLayer(nn.Module):
    def __init__(self, config: OlmoeConfig, layer_idx: int) -> None:
        super().__init__()
        self.self_attn = OlmoeAttention(config, layer_idx)
        self.mlp = OlmoeSparseMoeBlock(config)
        self.input_layernorm = OlmoeRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = OlmoeRMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states: Any, **kw: Any) -> Any:
        residual = hidden_states
        h = self.input_layernorm(hidden_states)
        h, _ = self.self_attn(h, **kw)
        hidden_states = residual + h
        residual = hidden_states
        h = self.post_attention_layernorm(hidden_states)
        h, _ = self.mlp(h)
        return residual + h


class StaticLayer:
    def __init__(self, max_len: int) -> None:
        self.max_len = max_len
        self.keys: Any = None
        self.values: Any = None
        self.is_initialized = False

    def lazy_initialization(self, key_states: Any) -> None:
        _, h, _, d = key_states.shape
        self.keys = torch.zeros((1, h, self.max_len, d), dtype=key_states.dtype, device=key_states.device)
        self.values = torch.zeros_like(self.keys)
        self.is_initialized = True

    def update(self, key_states: Any, value_states: Any, cache_kwargs: dict | None = None) -> tuple[Any, Any]:
        if not self.is_initialized:
            self.lazy_initialization(key_states)
        pos = (cache_kwargs or {}).get("cache_position")
        self.keys.index_copy_(2, pos, key_states)
        self.values.index_copy_(2, pos, value_states)
        return self.keys, self.values


class StaticCache:
    """Fixed-address KV cache: ``layers[i].keys/values`` are ``(1, heads, max_cache_len, head_dim)``;
    ``update`` is an ``index_copy_`` on dim 2 that returns the whole buffers; ``reset`` zeroes in place."""

    def __init__(self, config: OlmoeConfig, max_cache_len: int) -> None:
        self.max_cache_len = int(max_cache_len)
        self.layers = [StaticLayer(self.max_cache_len) for _ in range(config.num_hidden_layers)]

    def update(self, key_states: Any, value_states: Any, layer_idx: int, cache_kwargs: dict | None = None):
        return self.layers[layer_idx].update(key_states, value_states, cache_kwargs)

    def reset(self) -> None:
        for layer in self.layers:
            if layer.is_initialized:
                layer.keys.zero_()
                layer.values.zero_()


class OlmoeModel(nn.Module):
    def __init__(self, config: OlmoeConfig) -> None:
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([OlmoeDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = OlmoeRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.rotary_emb = OlmoeRotaryEmbedding(config)


class OlmoeForCausalLM(nn.Module):
    def __init__(self, config: OlmoeConfig) -> None:
        super().__init__()
        self.config = config
        self.model = OlmoeModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

    def forward(self, input_ids: Any, attention_mask: Any = None, past_key_values: Any = None, use_cache: bool = False,
                cache_position: Any = None, position_ids: Any = None, **kwargs: Any) -> Any:
        m = self.model
        x = m.embed_tokens(input_ids)
        bsz, q_len = input_ids.shape
        if cache_position is None:
            cache_position = torch.arange(q_len, device=x.device)
        if position_ids is None:
            position_ids = cache_position.unsqueeze(0)
        max_len = past_key_values.max_cache_len if past_key_values is not None else None
        cos, sin = m.rotary_emb(x, position_ids, max_len=max_len)
        mask4 = None
        if attention_mask is not None and attention_mask.dim() == 4:
            mask4 = attention_mask
        elif q_len > 1:
            kv_len = past_key_values.max_cache_len if past_key_values is not None else q_len
            neg = torch.finfo(x.dtype).min
            mask4 = torch.full((q_len, kv_len), neg, dtype=x.dtype, device=x.device)
            mask4 = mask4.masked_fill(torch.arange(kv_len, device=x.device)[None, :] <= cache_position[:, None], 0.0)
            mask4 = mask4[None, None]
        for layer in m.layers:
            x = layer(x, attention_mask=mask4, position_ids=position_ids, past_key_values=past_key_values,
                      use_cache=use_cache, cache_position=cache_position, position_embeddings=(cos, sin))
        x = m.norm(x)
        return SimpleNamespace(logits=self.lm_head(x), past_key_values=past_key_values)


def init_random_(model: OlmoeForCausalLM, seed: int = 0, std: float | None = None) -> OlmoeForCausalLM:
    """Seeded random init in place on the model's device: every matrix ``N(0, std)``, norm weights 1."""
    std = model.config.initializer_range if std is None else std
    dev = next(model.parameters()).device
    g = torch.Generator(device=dev).manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                p.copy_((torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * std).to(p.dtype))
    return model
