"""Llama-style decoder used by the benchmarks and end-to-end tests.

The reference ships no model; its benchmark configurations name Llama-3-8B,
a 1.1B Llama-style model, a 70B-architecture model and a tiny GPT.  This module
provides those architectures with random initialisation.  It is written for the
B200 training path: q/k/v and gate/up projections are single fused GEMMs, the
residual add is fused into RMSNorm, RoPE/SwiGLU/cross-entropy are single
kernels (``ops/model_ops.py``), attention goes through
``scaled_dot_product_attention`` and weight gradients can accumulate directly
into a flat gradient buffer (``main_grad``) owned by the ZeRO optimizer.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as Fnn
from torch import Tensor

from ..ops import model_ops as M


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    d_ff: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    max_seq_len: int = 4096
    activation_checkpointing: bool = False

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def num_params(self) -> int:
        hd = self.head_dim
        per_layer = (self.d_model * (self.n_heads + 2 * self.n_kv_heads) * hd + self.d_model * self.d_model
                     + 3 * self.d_model * self.d_ff + 2 * self.d_model)
        return self.n_layers * per_layer + 2 * self.vocab_size * self.d_model + self.d_model

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token: 6 x (matmul parameters) + causal attention."""
        hd = self.head_dim
        mat = self.n_layers * (self.d_model * (self.n_heads + 2 * self.n_kv_heads) * hd + self.d_model * self.d_model
                               + 3 * self.d_model * self.d_ff) + self.vocab_size * self.d_model
        attn = self.n_layers * 2 * seq_len * self.d_model  # QK^T and PV, halved for causality
        return 6.0 * mat + 6.0 * attn


PRESETS = {
    "llama3-8b": LlamaConfig(),
    "llama-1.1b": LlamaConfig(vocab_size=32000, d_model=2048, n_layers=22, n_heads=32, n_kv_heads=4, d_ff=5632,
                              rope_theta=10000.0, max_seq_len=2048),
    "llama3-70b": LlamaConfig(d_model=8192, n_layers=80, n_heads=64, n_kv_heads=8, d_ff=28672,
                              activation_checkpointing=True),
    "tiny": LlamaConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=4, n_kv_heads=2, d_ff=384,
                        rope_theta=10000.0, max_seq_len=128),
}


def get_config(name: str, **overrides) -> LlamaConfig:
    base = asdict(PRESETS[name])
    base.update(overrides)
    return LlamaConfig(**base)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: Tensor, residual: Optional[Tensor] = None):
        return M.rms_norm(x, self.weight, self.eps, residual)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.n_heads, self.n_kv, self.hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        self.wqkv = nn.Parameter(torch.empty((cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim, cfg.d_model))
        self.wo = nn.Parameter(torch.empty(cfg.d_model, cfg.n_heads * cfg.head_dim))

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        B, S, _ = x.shape
        qkv = M.linear(x, self.wqkv).view(B, S, self.n_heads + 2 * self.n_kv, self.hd)
        qkv = M.rope_qkv(qkv, cos, sin, self.n_heads + self.n_kv)
        # one split instead of three slices: its backward is a single concatenation of dq, dk, dv, where three slices
        # would each zero-fill a full qkv-sized tensor and autograd would then add them up (3 fills + 2 adds per layer)
        q, k, v = qkv.split([self.n_heads, self.n_kv, self.n_kv], dim=2)
        o = Fnn.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                             enable_gqa=self.n_kv != self.n_heads)
        return M.linear(o.transpose(1, 2).reshape(B, S, self.n_heads * self.hd), self.wo)


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.w_gate_up = nn.Parameter(torch.empty(2 * cfg.d_ff, cfg.d_model))
        self.w_down = nn.Parameter(torch.empty(cfg.d_model, cfg.d_ff))

    def forward(self, x: Tensor) -> Tensor:
        return M.linear(M.swiglu(M.linear(x, self.w_gate_up)), self.w_down)


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.attn = Attention(cfg)
        self.mlp_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.mlp = MLP(cfg)

    def forward(self, delta: Tensor, stream: Optional[Tensor], cos: Tensor, sin: Tensor):
        """``delta`` is the not-yet-added output of the previous sub-layer; ``stream`` the residual stream."""
        n, stream = self.attn_norm(delta, stream)
        a = self.attn(n, cos, sin)
        n, stream = self.mlp_norm(a, stream)
        return self.mlp(n), stream


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.final_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        self._rope = None
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, seed: int = 0, init: str = "scaled") -> None:
        """``init="scaled"``: N(0, 0.02) with the two output projections of every block divided by sqrt(2 * layers)
        (GPT-2 style residual scaling).  ``init="hf"``: N(0, 0.02) for every matrix, what
        ``transformers.LlamaForCausalLM`` does with its default ``initializer_range``."""
        if init not in ("scaled", "hf"):
            raise ValueError(f"unknown init scheme {init!r}")
        gen = torch.Generator(device="cpu").manual_seed(seed)
        std = 0.02
        for name, p in self.named_parameters():
            if p.dim() < 2:
                p.fill_(1.0)
            else:
                scale = std / math.sqrt(2 * self.cfg.n_layers) if (init == "scaled" and name.endswith(("wo", "w_down"))) else std
                if p.device.type == "cpu":
                    p.copy_(torch.randn(p.shape, generator=gen) * scale)
                else:
                    p.normal_(0.0, scale)

    def _tables(self, seq_len: int, device):
        if self._rope is None or self._rope[0].device != device or self._rope[0].shape[0] < seq_len:
            self._rope = M.rope_tables(max(seq_len, self.cfg.max_seq_len), self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    def hidden(self, tokens: Tensor) -> Tensor:
        cos, sin = self._tables(tokens.shape[1], tokens.device)
        delta, stream = self.embed(tokens), None
        for layer in self.layers:
            if self.cfg.activation_checkpointing and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                if stream is None:
                    stream = torch.zeros_like(delta)
                delta, stream = checkpoint(layer, delta, stream, cos, sin, use_reentrant=False)
            else:
                delta, stream = layer(delta, stream, cos, sin)
        out, _ = self.final_norm(delta, stream)
        return out

    def forward(self, tokens: Tensor, targets: Optional[Tensor] = None, loss_scale: float = 1.0):
        """Logits when ``targets`` is None, else the mean next-token loss times ``loss_scale``
        (``targets`` are already shifted)."""
        h = self.hidden(tokens)
        if targets is None:
            return M.linear(h, self.lm_head)
        B, S, D = h.shape
        return M.linear_cross_entropy(h.reshape(B * S, D), self.lm_head, targets.reshape(-1),
                                      main_grad=getattr(self.lm_head, "main_grad", None), loss_scale=loss_scale)


def build_llama(name_or_cfg, device="cpu", dtype=torch.float32, seed: int = 0, init: str = "scaled", **overrides) -> Llama:
    cfg = name_or_cfg if isinstance(name_or_cfg, LlamaConfig) else get_config(name_or_cfg, **overrides)
    with torch.device("meta"):
        model = Llama.__new__(Llama)
        nn.Module.__init__(model)
        model.cfg = cfg
        model.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        model.layers = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        model.final_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        model.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        model._rope = None
    model = model.to_empty(device=device).to(dtype)
    if torch.device(device).type == "cuda":
        torch.manual_seed(seed)
    model.reset_parameters(seed, init)
    return model


@torch.no_grad()
def load_hf_llama_weights(model: Llama, hf_state: dict) -> None:
    """Copy the weights of a ``transformers.LlamaForCausalLM`` state dict (``model.layers.N.self_attn.q_proj.weight``
    and so on) into ``model``: q/k/v are stacked into the fused ``wqkv`` (q heads first, then k, then v), gate/up into
    ``w_gate_up`` (gate first).  Both models use the rotate-half rotary convention, so no permutation is needed.
    Works in place, so parameters that an optimizer has already re-pointed into flat buffers stay where they are."""
    def take(name):
        return hf_state[name]

    model.embed.weight.copy_(take("model.embed_tokens.weight"))
    head = hf_state.get("lm_head.weight", hf_state["model.embed_tokens.weight"])       # tied embeddings: the same tensor
    model.lm_head.copy_(head)
    model.final_norm.weight.copy_(take("model.norm.weight"))
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}."
        layer.attn_norm.weight.copy_(take(pre + "input_layernorm.weight"))
        layer.mlp_norm.weight.copy_(take(pre + "post_attention_layernorm.weight"))
        q, k, v = (take(pre + f"self_attn.{n}_proj.weight") for n in ("q", "k", "v"))
        layer.attn.wqkv[: q.shape[0]].copy_(q)
        layer.attn.wqkv[q.shape[0]: q.shape[0] + k.shape[0]].copy_(k)
        layer.attn.wqkv[q.shape[0] + k.shape[0]:].copy_(v)
        layer.attn.wo.copy_(take(pre + "self_attn.o_proj.weight"))
        gate, up = take(pre + "mlp.gate_proj.weight"), take(pre + "mlp.up_proj.weight")
        layer.mlp.w_gate_up[: gate.shape[0]].copy_(gate)
        layer.mlp.w_gate_up[gate.shape[0]:].copy_(up)
        layer.mlp.w_down.copy_(take(pre + "mlp.down_proj.weight"))
