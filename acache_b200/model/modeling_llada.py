"""LLaDA-8B architecture for paged serving.

Llama-style pre-norm block with separate q/k/v projections, RoPE computed in fp32,
SiLU-gated FFN and an untied output head; ragged ``[n]`` and batched ``[B, T]`` inputs
(reference: nano-vdllm/model/modeling_llada.py:593-767 block, :889-982 model,
:999-1064 wrapper).  Parameter names equal the reference's, so its checkpoints load
with ``load_state_dict``.  Projections, normalisation, RoPE + K/V scatter, attention and the
gated activation are this package's kernels (``modeling_common.OWN_GEMM`` sends the
projections to the library GEMM instead).
"""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..utils import get_context
from .attention import Attention
from .configuration import LLaDAConfig
from . import modeling_common as mc
from .modeling_common import FusedProjections, RMSNorm, RopeCache, concat_gate_up, dense_pending, gated_mlp_input, project_qkv, select_pending


class LLaDALlamaBlock(nn.Module):
    def __init__(self, layer_id: int, config: LLaDAConfig, rope: RopeCache, device=None, dtype=None):
        super().__init__()
        self.layer_id = layer_id
        self.config = config
        d, kvd, ffn = config.d_model, config.effective_n_kv_heads * (config.d_model // config.n_heads), config.ffn_size
        kw = dict(device=device, dtype=dtype)
        qkv_bias = config.include_bias or config.include_qkv_bias
        self.attn_norm = RMSNorm(d, config.rms_norm_eps, **kw)
        self.ff_norm = RMSNorm(d, config.rms_norm_eps, **kw)
        self.q_proj = nn.Linear(d, d, bias=qkv_bias, **kw)
        self.k_proj = nn.Linear(d, kvd, bias=qkv_bias, **kw)
        self.v_proj = nn.Linear(d, kvd, bias=qkv_bias, **kw)
        self.attn_out = nn.Linear(d, d, bias=config.include_bias, **kw)
        self.ff_proj = nn.Linear(d, ffn, bias=config.include_bias, **kw)
        self.up_proj = nn.Linear(d, ffn, bias=config.include_bias, **kw)
        self.ff_out = nn.Linear(ffn, d, bias=config.include_bias, **kw)
        self.rotary_emb = rope
        self.attn = Attention(num_heads=config.n_heads, head_dim=d // config.n_heads,
                              num_kv_heads=config.effective_n_kv_heads)
        self._qkv_w = self._qkv_b = self._gate_up_w = None
        self._fused = FusedProjections()

    def _projection_params(self):
        return (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self.q_proj.bias, self.ff_proj.weight,
                self.up_proj.weight)

    def fuse_qkv(self):
        """One projection GEMM for q, k and v: the three weights become views of one
        buffer (state-dict names and values are unchanged)."""
        w = torch.cat([self.q_proj.weight.data, self.k_proj.weight.data, self.v_proj.weight.data], dim=0)
        d, kvd = self.q_proj.out_features, self.k_proj.out_features
        self.q_proj.weight.data, self.k_proj.weight.data, self.v_proj.weight.data = w[:d], w[d:d + kvd], w[d + kvd:]
        self._qkv_w = w
        if self.q_proj.bias is not None:
            b = torch.cat([self.q_proj.bias.data, self.k_proj.bias.data, self.v_proj.bias.data])
            self.q_proj.bias.data, self.k_proj.bias.data, self.v_proj.bias.data = b[:d], b[d:d + kvd], b[d + kvd:]
            self._qkv_b = b
        self._gate_up_w = concat_gate_up(self.ff_proj, self.up_proj) if self.ff_proj.bias is None else None
        self._fused.reset(self._projection_params())

    def forward(self, x: torch.Tensor, position_ids: torch.Tensor, max_pos: int, delta=None):
        """``x [n, d]`` rows of the ragged batch (updated in place), ``position_ids [n]`` int64;
        ``delta`` is the previous block's feed-forward output, still to be added to ``x``.
        Returns ``(x, delta)`` with this block's feed-forward output pending in the same way, so
        that every residual add is fused into the normalisation that follows it."""
        cfg = self.config
        n = x.shape[0]
        nh, hkv, D = cfg.n_heads, cfg.effective_n_kv_heads, cfg.d_model // cfg.n_heads
        h = self.attn_norm(x, delta)
        cos, sin = self.rotary_emb.get(max_pos, x.device)
        ctx = get_context()
        attn = self.attn
        if (self._qkv_w is None or self._qkv_w.data_ptr() != self.q_proj.weight.data_ptr()
                or self._fused.stale(self._projection_params())):
            self.fuse_qkv()      # first use, or the parameters were replaced since (load, cast, move)
        q, k, v = project_qkv(h, self._qkv_w, self._qkv_b, nh, hkv, D, position_ids, cos, sin, attn, ctx, self._fused)
        att = attn(q, k, v).reshape(n, nh * D)
        attn.kv_already_stored = False
        h = self.ff_norm(x, dense_pending(att, self.attn_out.weight, self.attn_out.bias))
        h = gated_mlp_input(h, self._fused, self.ff_proj, self.up_proj, cfg.activation_type, self._gate_up_w)
        return x, dense_pending(h, self.ff_out.weight, self.ff_out.bias)


class LLaDAModel(nn.Module):
    def __init__(self, config: LLaDAConfig, device=None, dtype=None):
        super().__init__()
        self.config = config
        kw = dict(device=device, dtype=dtype)
        D = config.d_model // config.n_heads
        self.rope = RopeCache(D, config.rope_theta, torch.float32)
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.embedding_size or config.vocab_size, config.d_model, **kw),
            ln_f=RMSNorm(config.d_model, config.rms_norm_eps, **kw),
        ))
        self.transformer.update({"blocks": nn.ModuleList(
            [LLaDALlamaBlock(i, config, self.rope, **kw) for i in range(config.n_layers)])})
        if not config.weight_tying:
            self.transformer.update({"ff_out": nn.Linear(config.d_model, config.embedding_size or config.vocab_size,
                                                         bias=config.include_bias, **kw)})

    def forward(self, input_ids, position_ids=None, output_hidden_states=None, compute_logits=True,
                logits_keep_indices=None, max_pos: int | None = None, greedy_stats: bool = False):
        """``greedy_stats``: the caller only needs the arg-max token and its confidence of every
        kept row; when the fused output head can serve that, ``.stats = (x0, confidence)`` (flat,
        one entry per row) is returned and ``.logits`` is None (the logits are never written)."""
        shape = input_ids.shape
        ids = input_ids.reshape(-1)
        if position_ids is None:
            position_ids = torch.arange(ids.numel(), device=ids.device)
        pos = position_ids.reshape(-1)
        if max_pos is None:
            max_pos = int(pos.max().item()) + 1
        x = self.transformer["wte"](ids)
        if self.config.input_emb_norm:
            x = x * (self.config.d_model ** 0.5)
        delta = None
        for block in self.transformer["blocks"]:
            x, delta = block(x, pos, max_pos, delta)
        logits = None
        if compute_logits:
            if logits_keep_indices is not None:
                x = x.index_select(0, logits_keep_indices)
                delta = select_pending(delta, logits_keep_indices)
            x = self.transformer["ln_f"](x, delta)
            head = self.transformer["wte"] if self.config.weight_tying else self.transformer["ff_out"]
            if (greedy_stats and mc.OWN_HEAD and getattr(head, "bias", None) is None and not self.config.scale_logits
                    and ops._gemm_ok(x, head.weight)):
                return SimpleNamespace(logits=None, stats=ops.linear_argmax(x, head.weight), hidden_states=None)
            if mc.OWN_HEAD and ops._gemm_ok(x, head.weight):
                logits = ops.linear(x, head.weight, getattr(head, "bias", None))
            else:
                logits = F.linear(x, head.weight, getattr(head, "bias", None))
            if self.config.scale_logits:
                logits = logits * (self.config.d_model ** -0.5)
            if logits_keep_indices is None:
                logits = logits.view(*shape, -1)
        return SimpleNamespace(logits=logits, stats=None, hidden_states=None)


class LLaDAModelLM(nn.Module):
    """Wrapper with the reference's attribute layout: ``.model`` is the transformer,
    ``.config`` the architecture (reference: modeling_llada.py:999-1064)."""

    def __init__(self, config: LLaDAConfig, device=None, dtype=None, init_params: bool = True, seed: int | None = None):
        super().__init__()
        self.config = config
        self.model = LLaDAModel(config, device=device, dtype=dtype)
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
            if name.endswith("norm.weight") or name.endswith("ln_f.weight"):
                p.fill_(1.0)
            elif name.endswith(".bias"):
                p.zero_()
            else:
                p.normal_(0.0, self.config.init_std, generator=gen)

    def fuse_projections(self):
        for block in self.model.transformer["blocks"]:
            block.fuse_qkv()
        return self

    def forward(self, input_ids=None, output_hidden_states=None, position_ids=None, logits_keep_indices=None,
                compute_logits=True, max_pos=None, greedy_stats=False):
        return self.model(input_ids, position_ids=position_ids, compute_logits=compute_logits,
                          logits_keep_indices=logits_keep_indices, max_pos=max_pos, greedy_stats=greedy_stats)
