"""Decoder-only causal LM (Qwen3 and Llama-3 families) on the library's own kernels.

Module and parameter names are the Hugging Face ones (``model.embed_tokens``,
``model.layers.{i}.self_attn.{q,k,v,o}_proj``, ``self_attn.{q,k}_norm``, ``mlp.{gate,up,down}_proj``,
``input_layernorm``, ``post_attention_layernorm``, ``model.norm``, ``lm_head``), so the optimizer
factory's name filters, the bank schemes and ``save_pretrained`` checkpoints behave as they do for the
HF models the reference trains (``src/himuon/model.py:7-20``).  The reference runs HF
``transformers`` modules on PyTorch library kernels; here every op of the forward and backward pass
is an sm_100a kernel from :mod:`himuon_b200.ops` when the model is bf16 on a CUDA device.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..ops import reference as ref
from .config import DecoderConfig


class Linear(nn.Linear):
    """``nn.Linear`` whose matmuls run on the tcgen05 GEMM (forward, dgrad and wgrad)."""

    def forward(self, x):
        y = ops.linear(x, self.weight)
        return y if self.bias is None else y + self.bias


def _bank_pair(first: nn.Linear, second: nn.Linear):
    """When two bias-free projections occupy neighbouring slots ``2i, 2i+1`` of one parameter bank that a
    sharding engine serves, returns a callable computing both with a single GEMM; otherwise ``None``."""
    name = getattr(first, "_bank_name", None)
    if name is None or getattr(second, "_bank_name", None) != name or first.bias is not None or second.bias is not None:
        return None
    engine = getattr(getattr(first, "_bank_root", None), "_bank_engine", None)
    if engine is None or second._bank_idx != first._bank_idx + 1 or not hasattr(engine, "linear_pair"):
        return None
    return lambda x: engine.linear_pair(x, name, first._bank_idx)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.variance_epsilon, defer_dw=True)


class Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        H, D = cfg.hidden_size, cfg.head_dim
        self.q_proj = Linear(H, cfg.num_attention_heads * D, bias=False)
        self.k_proj = Linear(H, cfg.num_key_value_heads * D, bias=False)
        self.v_proj = Linear(H, cfg.num_key_value_heads * D, bias=False)
        self.o_proj = Linear(cfg.num_attention_heads * D, H, bias=False)
        if cfg.qk_norm:
            self.q_norm = RMSNorm(D, cfg.rms_norm_eps)
            self.k_norm = RMSNorm(D, cfg.rms_norm_eps)

    def forward(self, x2d, B: int, S: int, cos_sin):
        cfg = self.cfg
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        q = self.q_proj(x2d)
        pair = _bank_pair(self.k_proj, self.v_proj)
        if pair is not None:
            kv = pair(x2d)                      # k and v are neighbouring bank slots: one GEMM, column-sliced
            k, v = ops.split_cols(kv, Hkv * D)
        else:
            k = self.k_proj(x2d)
            v = self.v_proj(x2d)
        qw = self.q_norm.weight if cfg.qk_norm else None
        kw = self.k_norm.weight if cfg.qk_norm else None
        q = ops.head_norm_rope(q, qw, cos_sin, Hq, S, D, cfg.rms_norm_eps, defer_dw=True, inplace_grad=True)
        k = ops.head_norm_rope(k, kw, cos_sin, Hkv, S, D, cfg.rms_norm_eps, defer_dw=True, inplace_grad=True)
        o = ops.attention(q, k, v, B, S, Hq, Hkv, D)
        return self.o_proj(o)


class MLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.gate_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x2d):
        pair = _bank_pair(self.gate_proj, self.up_proj)
        if pair is not None:
            return self.down_proj(ops.swiglu_packed(pair(x2d)))
        return self.down_proj(ops.swiglu(self.gate_proj(x2d), self.up_proj(x2d)))


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.self_attn = Attention(cfg)
        self.mlp = MLP(cfg)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, h2d, delta, B: int, S: int, cos_sin):
        """``delta`` is the previous block's output that has not been added to the residual stream yet (``None``
        for the first layer): every residual add is fused with the RMSNorm that follows it.  Returns the updated
        stream and this layer's own pending MLP output."""
        h2d, n1 = ops.add_rmsnorm(h2d, delta, self.input_layernorm.weight, self.input_layernorm.variance_epsilon, defer_dw=True)
        a = self.self_attn(n1, B, S, cos_sin)
        h2d, n2 = ops.add_rmsnorm(h2d, a, self.post_attention_layernorm.weight,
                                      self.post_attention_layernorm.variance_epsilon, defer_dw=True)
        return h2d, self.mlp(n2)


class DecoderModel(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(DecoderLayer(cfg) for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


@dataclass
class CausalLMOutput:
    loss: torch.Tensor | None
    logits: torch.Tensor | None


class CausalLM(nn.Module):
    """``Qwen3ForCausalLM`` / ``LlamaForCausalLM`` equivalent with random initialisation."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.config = cfg
        self.config.use_cache = False
        self.model = DecoderModel(cfg)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.gradient_checkpointing = False
        self.loss_scale: float | None = None   # set by the training loop to 1/grad_accumulation
        self._rope_cache: dict = {}
        self.apply(self._init_weights)

    def _init_weights(self, m):
        std = self.config.initializer_range
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=std)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=std)

    # -- HF-style switches --------------------------------------------------------------------
    def gradient_checkpointing_enable(self, **_):
        self.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.gradient_checkpointing = False

    def set_loss_scale(self, scale: float | None):
        """Tell the fused lm_head + cross-entropy which factor multiplies the loss before
        ``backward()`` so the head's weight gradient can be accumulated in place."""
        self.loss_scale = scale

    def _rope(self, S: int, device):
        key = (S, str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = ref.rope_tables(S, self.config.head_dim, self.config.rope_theta, device=device)
        return self._rope_cache[key]

    def hidden_states(self, input_ids):
        B, S = input_ids.shape
        cos_sin = self._rope(S, input_ids.device)
        h = ops.embedding(input_ids, self.model.embed_tokens.weight).reshape(B * S, -1)
        delta = None
        # an engine that stages weights or reduces gradients per layer group is told where the layer loop stands
        engine = getattr(self, "_layer_hooks", None)
        fenced = engine is not None
        for i, layer in enumerate(self.model.layers):
            if fenced:
                h, delta = engine.pre_layer(i, h, delta)
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                h, delta = checkpoint(layer, h, delta, B, S, cos_sin, use_reentrant=False)
            else:
                h, delta = layer(h, delta, B, S, cos_sin)
            if fenced:
                h, delta = engine.post_layer(i, h, delta)
        return ops.add_rmsnorm(h, delta, self.model.norm.weight, self.model.norm.variance_epsilon, defer_dw=True)[1]

    def forward(self, input_ids, attention_mask=None, labels=None, return_logits: bool = False, **_):
        """Causal LM forward.  With ``labels`` the shifted mean token cross-entropy is returned as
        ``.loss`` and, unless ``return_logits`` is set, logits are never materialised.  ``attention_mask``
        is accepted for API compatibility; attention is causal and padding is not masked."""
        B, S = input_ids.shape
        h = self.hidden_states(input_ids)
        loss, logits = None, None
        if labels is not None:
            shifted = torch.full_like(labels, -100)
            shifted[:, :-1] = labels[:, 1:]
            head = self._head_weight()
            # in-forward accumulation of the head's weight gradient only when a backward pass follows this forward
            scale = self.loss_scale if (self.training and torch.is_grad_enabled()) else None
            loss = ops.linear_cross_entropy(h, head[0], shifted.reshape(-1), sink=head[1], loss_scale=scale)
        if labels is None or return_logits:
            logits = ops.linear(h, self._head_weight()[0]).view(B, S, -1)
        return CausalLMOutput(loss=loss, logits=logits)

    def _head_weight(self):
        return self.lm_head.weight, None

    # -- checkpoint I/O -----------------------------------------------------------------------
    def save_pretrained(self, save_directory: str, state_dict: dict | None = None, **_):
        """Write ``config.json`` + ``model.safetensors`` in the Hugging Face layout."""
        from safetensors.torch import save_file

        os.makedirs(save_directory, exist_ok=True)
        sd = state_dict if state_dict is not None else self.state_dict()
        out = {}
        for k, v in sd.items():
            if self.config.tie_word_embeddings and k == "lm_head.weight":
                continue
            out[k] = v.detach().to("cpu").contiguous()
        save_file(out, os.path.join(save_directory, "model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(save_directory, "config.json"), "w") as f:
            json.dump(self.config.to_hf_dict(), f, indent=2)

    @classmethod
    def from_pretrained(cls, directory: str, cfg: DecoderConfig | None = None):
        from safetensors.torch import load_file

        if cfg is None:
            with open(os.path.join(directory, "config.json")) as f:
                d = json.load(f)
            cfg = DecoderConfig(
                model_type=d.get("model_type", "qwen3"), vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
                intermediate_size=d["intermediate_size"], num_hidden_layers=d["num_hidden_layers"],
                num_attention_heads=d["num_attention_heads"], num_key_value_heads=d["num_key_value_heads"],
                head_dim=d.get("head_dim", d["hidden_size"] // d["num_attention_heads"]),
                rms_norm_eps=d["rms_norm_eps"], rope_theta=d.get("rope_theta", 10000.0),
                tie_word_embeddings=d.get("tie_word_embeddings", False),
                max_position_embeddings=d.get("max_position_embeddings", 2048))
        model = cls(cfg)
        sd = load_file(os.path.join(directory, "model.safetensors"))
        if cfg.tie_word_embeddings:
            sd.setdefault("lm_head.weight", sd["model.embed_tokens.weight"])
        model.load_state_dict(sd)
        return model
