"""Dense CPU forward of the two served architectures, one request at a time.

LLaDA (Llama-style block, separate q/k/v projections, SiLU-gated FFN, untied
output head): reference nano-vdllm/model/modeling_llada.py:308-323 (RMSNorm in
fp32, cast back, times weight), :412-453 (RoPE in fp32), :717-767 (block),
:889-982 (model).  Dream (Qwen2.5-style GQA with QKV bias): reference
nano-vdllm/model/modeling_dream.py:76-81 (RMSNorm), :159-170,472-476 (RoPE with
the table cast to the activation dtype), :297-303 (MLP), :827-896 (model).

The state dict uses the reference's parameter names, so the same tensors load
into the served model and into this restatement.
"""
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .rope import dream_rope_qk, llada_rope_qk


@dataclass
class ArchSpec:
    kind: str  # 'llada' | 'dream'
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    ffn: int
    vocab: int
    rope_theta: float
    rms_eps: float
    act: str = "silu"
    mask_id: int = 126336

    @property
    def head_dim(self):
        return self.d_model // self.n_heads


def _act(name):
    return {"silu": F.silu, "relu": F.relu, "gelu": F.gelu}[name]


def _rmsnorm(x, w, eps):
    dt = x.dtype
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return w * xf.to(dt)


class KVState:
    """Per-request dense logical cache: K (post-RoPE) and V per layer, one row per
    logical position."""

    def __init__(self, spec: ArchSpec, length: int, dtype):
        shape = (spec.n_layers, length, spec.n_kv_heads, spec.head_dim)
        self.k = torch.zeros(shape, dtype=dtype)
        self.v = torch.zeros(shape, dtype=dtype)


class OracleModel:
    def __init__(self, spec: ArchSpec, state_dict: dict, dtype=torch.float32):
        self.spec = spec
        self.dtype = dtype
        self.w = {k: v.to(dtype) for k, v in state_dict.items()}

    # -- parameter access by role ---------------------------------------------
    def _p(self, layer, role):
        s = self.spec
        if s.kind == "llada":
            base = f"model.transformer.blocks.{layer}."
            name = {
                "ln1": "attn_norm.weight", "ln2": "ff_norm.weight",
                "q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "attn_out",
                "gate": "ff_proj", "up": "up_proj", "down": "ff_out",
            }[role]
        else:
            base = f"model.layers.{layer}."
            name = {
                "ln1": "input_layernorm.weight", "ln2": "post_attention_layernorm.weight",
                "q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
                "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj",
            }[role]
        if role in ("ln1", "ln2"):
            return self.w[base + name]
        return self.w[base + name + ".weight"], self.w.get(base + name + ".bias")

    def _lin(self, x, layer, role):
        w, b = self._p(layer, role)
        return F.linear(x, w, b)

    def embed(self, tokens):
        key = "model.transformer.wte.weight" if self.spec.kind == "llada" else "model.embed_tokens.weight"
        return self.w[key][tokens]

    def head(self, x):
        if self.spec.kind == "llada":
            x = _rmsnorm(x, self.w["model.transformer.ln_f.weight"], self.spec.rms_eps)
            return F.linear(x, self.w["model.transformer.ff_out.weight"])
        x = _rmsnorm(x, self.w["model.norm.weight"], self.spec.rms_eps)
        return F.linear(x, self.w["lm_head.weight"])

    # -- one forward over a set of rows of one request -----------------------------
    def forward_rows(self, tokens, positions, kv: KVState, write_idx, logits_rows=None, probe=None):
        """tokens/positions: int64 [n] (the query rows, logical positions);
        write_idx: int64 [n] rows of ``kv`` that receive this forward's K/V
        (normally == positions; -1 = do not store this row).  Attention of every row is over ALL rows of
        ``kv`` (bidirectional).  ``probe``: optional dict with 'mask_rows'
        (bool [n]), 'affix' (slice of kv rows) and 'acc' (fp32 [A]) to
        accumulate the anchor influence score of every layer
        (reference: nano-vdllm/model_runner.py:730-773).
        Returns logits [len(logits_rows), vocab] or None."""
        s = self.spec
        nh, hkv, D = s.n_heads, s.n_kv_heads, s.head_dim
        g = nh // hkv
        scale = D ** -0.5
        act = _act(s.act)
        x = self.embed(tokens)
        n = tokens.shape[0]
        for l in range(s.n_layers):
            h = _rmsnorm(x, self._p(l, "ln1"), s.rms_eps)
            q = self._lin(h, l, "q").view(n, nh, D)
            k = self._lin(h, l, "k").view(n, hkv, D)
            v = self._lin(h, l, "v").view(n, hkv, D)
            if s.kind == "llada":
                q, k = llada_rope_qk(q, k, positions, s.rope_theta)
            else:
                q, k = dream_rope_qk(q, k, positions, s.rope_theta)
            if probe is not None and bool(probe["mask_rows"].any()):
                from .importance import layer_importance
                probe["acc"] += layer_importance(q[probe["mask_rows"]], kv.k[l, probe["affix"]], scale,
                                                 exact=probe.get("exact", False))
            keep = write_idx >= 0      # -1: the row is only queried, its cached K/V stays
            kv.k[l, write_idx[keep]] = k[keep]
            kv.v[l, write_idx[keep]] = v[keep]
            kf = kv.k[l].float().permute(1, 2, 0).repeat_interleave(g, dim=0)
            vf = kv.v[l].float().permute(1, 0, 2).repeat_interleave(g, dim=0)
            w = torch.softmax((q.float().permute(1, 0, 2) @ kf) * scale, dim=-1)
            att = (w @ vf).permute(1, 0, 2).to(x.dtype).reshape(n, nh * D)
            x = x + self._lin(att, l, "o")
            h = _rmsnorm(x, self._p(l, "ln2"), s.rms_eps)
            x = x + self._lin(act(self._lin(h, l, "gate")) * self._lin(h, l, "up"), l, "down")
        if logits_rows is None:
            return None
        return self.head(x[logits_rows])


def random_state_dict(spec: ArchSpec, seed: int, std: float = 0.02, dtype=torch.float32):
    """Random-init weights with the reference's parameter names (normal(0, std),
    norm weights 1, Dream QKV biases normal(0, std))."""
    g = torch.Generator().manual_seed(seed)

    def rn(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    kvd = spec.n_kv_heads * spec.head_dim
    sd = {}
    if spec.kind == "llada":
        sd["model.transformer.wte.weight"] = rn(spec.vocab, spec.d_model)
        for l in range(spec.n_layers):
            b = f"model.transformer.blocks.{l}."
            sd[b + "attn_norm.weight"] = torch.ones(spec.d_model, dtype=dtype)
            sd[b + "ff_norm.weight"] = torch.ones(spec.d_model, dtype=dtype)
            sd[b + "q_proj.weight"] = rn(spec.d_model, spec.d_model)
            sd[b + "k_proj.weight"] = rn(kvd, spec.d_model)
            sd[b + "v_proj.weight"] = rn(kvd, spec.d_model)
            sd[b + "attn_out.weight"] = rn(spec.d_model, spec.d_model)
            sd[b + "ff_proj.weight"] = rn(spec.ffn, spec.d_model)
            sd[b + "up_proj.weight"] = rn(spec.ffn, spec.d_model)
            sd[b + "ff_out.weight"] = rn(spec.d_model, spec.ffn)
        sd["model.transformer.ln_f.weight"] = torch.ones(spec.d_model, dtype=dtype)
        sd["model.transformer.ff_out.weight"] = rn(spec.vocab, spec.d_model)
    else:
        sd["model.embed_tokens.weight"] = rn(spec.vocab, spec.d_model)
        for l in range(spec.n_layers):
            b = f"model.layers.{l}."
            sd[b + "input_layernorm.weight"] = torch.ones(spec.d_model, dtype=dtype)
            sd[b + "post_attention_layernorm.weight"] = torch.ones(spec.d_model, dtype=dtype)
            sd[b + "self_attn.q_proj.weight"] = rn(spec.d_model, spec.d_model)
            sd[b + "self_attn.q_proj.bias"] = rn(spec.d_model)
            sd[b + "self_attn.k_proj.weight"] = rn(kvd, spec.d_model)
            sd[b + "self_attn.k_proj.bias"] = rn(kvd)
            sd[b + "self_attn.v_proj.weight"] = rn(kvd, spec.d_model)
            sd[b + "self_attn.v_proj.bias"] = rn(kvd)
            sd[b + "self_attn.o_proj.weight"] = rn(spec.d_model, spec.d_model)
            sd[b + "mlp.gate_proj.weight"] = rn(spec.ffn, spec.d_model)
            sd[b + "mlp.up_proj.weight"] = rn(spec.ffn, spec.d_model)
            sd[b + "mlp.down_proj.weight"] = rn(spec.d_model, spec.ffn)
        sd["model.norm.weight"] = torch.ones(spec.d_model, dtype=dtype)
        sd["lm_head.weight"] = rn(spec.vocab, spec.d_model)
    # A random output head can make the mask token itself the arg-max, and block decoding
    # (here and in the reference) only ends when no mask is left.  Giving the mask row the
    # weights of row 0 makes the two logits equal, and arg-max ties go to the lower index.
    head = "model.transformer.ff_out.weight" if spec.kind == "llada" else "lm_head.weight"
    if 0 < spec.mask_id < spec.vocab:
        sd[head][spec.mask_id] = sd[head][0]
    return sd
