"""Dream-7B architecture (Qwen2.5-style GQA with QKV bias) for paged serving.

reference: nano-vdllm/model/modeling_dream.py:76-81 (RMSNorm), :159-170 (RoPE tables cast
to the activation dtype), :297-303 (MLP), :439-501 (attention), :827-896 (model with
``logits_keep_indices`` row selection before the output head).  Parameter names equal
the reference's.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..utils import get_context
from .attention import Attention
from .configuration import DreamConfig
from . import modeling_common as mc
from .modeling_common import FusedProjections, RMSNorm, RopeCache, concat_gate_up, dense_pending, gated_mlp_input, project_qkv, select_pending


class DreamMLP(nn.Module):
    def __init__(self, config: DreamConfig, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False, **kw)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False, **kw)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False, **kw)
        self.act = config.hidden_act
        self._fused = FusedProjections()
        self._gate_up_w = None

    def _params(self):
        return (self.gate_proj.weight, self.up_proj.weight)

    def forward(self, x):
        if (self._gate_up_w is None or self._gate_up_w.data_ptr() != self.gate_proj.weight.data_ptr()
                or self._fused.stale(self._params())):
            self._gate_up_w = concat_gate_up(self.gate_proj, self.up_proj)
            self._fused.reset(self._params())
        h = gated_mlp_input(x, self._fused, self.gate_proj, self.up_proj, self.act, self._gate_up_w)
        return dense_pending(h, self.down_proj.weight)


class DreamSdpaAttention(nn.Module):
    def __init__(self, config: DreamConfig, layer_idx: int, rope: RopeCache, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.config = config
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=True, **kw)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=True, **kw)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=True, **kw)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=False, **kw)
        self.rotary_emb = rope
        self.attn = Attention(num_heads=self.num_heads, head_dim=self.head_dim, num_kv_heads=self.num_key_value_heads)
        self._qkv_w = self._qkv_b = None
        self._fused = FusedProjections()

    def _projection_params(self):
        return (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self.q_proj.bias, self.k_proj.bias,
                self.v_proj.bias)

    def fuse_qkv(self):
        w = torch.cat([self.q_proj.weight.data, self.k_proj.weight.data, self.v_proj.weight.data], dim=0)
        b = torch.cat([self.q_proj.bias.data, self.k_proj.bias.data, self.v_proj.bias.data])
        d, kvd = self.q_proj.out_features, self.k_proj.out_features
        self.q_proj.weight.data, self.k_proj.weight.data, self.v_proj.weight.data = w[:d], w[d:d + kvd], w[d + kvd:]
        self.q_proj.bias.data, self.k_proj.bias.data, self.v_proj.bias.data = b[:d], b[d:d + kvd], b[d + kvd:]
        self._qkv_w, self._qkv_b = w, b
        self._fused.reset(self._projection_params())

    def forward(self, x, position_ids, max_pos):
        n = x.shape[0]
        nh, hkv, D = self.num_heads, self.num_key_value_heads, self.head_dim
        cos, sin = self.rotary_emb.get(max_pos, x.device)
        ctx = get_context()
        attn = self.attn
        if (self._qkv_w is None or self._qkv_w.data_ptr() != self.q_proj.weight.data_ptr()
                or self._fused.stale(self._projection_params())):
            self.fuse_qkv()      # first use, or the parameters were replaced since (load, cast, move)
        q, k, v = project_qkv(x, self._qkv_w, self._qkv_b, nh, hkv, D, position_ids, cos, sin, attn, ctx, self._fused)
        o = attn(q, k, v).reshape(n, nh * D)
        attn.kv_already_stored = False
        return dense_pending(o, self.o_proj.weight)


class DreamDecoderLayer(nn.Module):
    def __init__(self, config: DreamConfig, layer_idx: int, rope: RopeCache, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.self_attn = DreamSdpaAttention(config, layer_idx, rope, **kw)
        self.mlp = DreamMLP(config, **kw)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, **kw)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, **kw)

    def forward(self, x, position_ids, max_pos, delta=None):
        """Returns ``(x, delta)``: ``x`` is updated in place, the MLP output is left pending so the
        next normalisation adds it (residual add fused into the norm kernel)."""
        h = self.input_layernorm(x, delta)
        h = self.post_attention_layernorm(x, self.self_attn(h, position_ids, max_pos))
        return x, self.mlp(h)


class DreamBaseModel(nn.Module):
    def __init__(self, config: DreamConfig, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.config = config
        D = config.hidden_size // config.num_attention_heads
        # the reference casts the fp32 cos/sin to the activation dtype before use
        self.rope = RopeCache(D, config.rope_theta, dtype or torch.float32)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, **kw)
        self.layers = nn.ModuleList([DreamDecoderLayer(config, i, self.rope, **kw) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, **kw)


class DreamModel(nn.Module):
    """``.model`` holds the decoder, ``.lm_head`` the output projection
    (reference: modeling_dream.py:827-896)."""

    def __init__(self, config: DreamConfig, device=None, dtype=None, init_params: bool = True, seed: int | None = None):
        super().__init__()
        self.config = config
        self.model = DreamBaseModel(config, device=device, dtype=dtype)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False, device=device, dtype=dtype)
        if init_params:
            self.reset_parameters(seed)
        for p in self.parameters():  # serving only: no autograd state
            p.requires_grad_(False)

    @property
    def device(self):
        return next(self.parameters()).device

    @torch.no_grad()
    def reset_parameters(self, seed: int | None = None):
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if "layernorm" in name or name.endswith("model.norm.weight"):
                p.fill_(1.0)
            else:
                p.normal_(0.0, self.config.initializer_range, generator=gen)

    def fuse_projections(self):
        for layer in self.model.layers:
            layer.self_attn.fuse_qkv()
        return self

    def forward(self, input_ids=None, position_ids=None, compute_logits=True, logits_keep_indices=None, max_pos=None,
                greedy_stats=False, **_unused):
        """``greedy_stats``: see ``LLaDAModel.forward``."""
        shape = input_ids.shape
        ids = input_ids.reshape(-1)
        if position_ids is None:
            position_ids = torch.arange(ids.numel(), device=ids.device)
        pos = position_ids.reshape(-1)
        if max_pos is None:
            max_pos = int(pos.max().item()) + 1
        x = self.model.embed_tokens(ids)
        delta = None
        for layer in self.model.layers:
            x, delta = layer(x, pos, max_pos, delta)
        logits = None
        if compute_logits:
            if logits_keep_indices is not None:
                x = x.index_select(0, logits_keep_indices)
                delta = select_pending(delta, logits_keep_indices)
            x = self.model.norm(x, delta)
            if greedy_stats and mc.OWN_HEAD and ops._gemm_ok(x, self.lm_head.weight):
                return SimpleNamespace(logits=None, stats=ops.linear_argmax(x, self.lm_head.weight), hidden_states=None)
            if mc.OWN_HEAD and ops._gemm_ok(x, self.lm_head.weight):
                logits = ops.linear(x, self.lm_head.weight)
            else:
                logits = F.linear(x, self.lm_head.weight)
            if logits_keep_indices is None:
                logits = logits.view(*shape, -1)
        return SimpleNamespace(logits=logits, stats=None, hidden_states=None)
