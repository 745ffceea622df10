"""Architecture descriptions of the two served model families.

Field names follow the reference configuration classes so that code reading them
(the engine's KV-cache sizing, state-dict loaders) is unchanged: LLaDA
(reference: nano-vdllm/model/configuration_llada.py:150-381) and Dream
(reference: nano-vdllm/model/configuration_dream.py).  They are plain
dataclasses; any object with the same attributes works.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class LLaDAConfig:
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int | None = 32
    n_layers: int = 32
    mlp_hidden_size: int | None = 12288
    mlp_ratio: int = 4
    activation_type: str = "silu"
    block_type: str = "llama"
    block_group_size: int = 1
    rope: bool = True
    rope_full_precision: bool = True
    rope_theta: float = 500000.0
    rms_norm_eps: float = 1e-5
    layer_norm_type: str = "rms"
    include_bias: bool = False
    include_qkv_bias: bool = False
    weight_tying: bool = False
    input_emb_norm: bool = False
    scale_logits: bool = False
    vocab_size: int = 126464
    embedding_size: int | None = 126464
    max_sequence_length: int = 4096
    train_max_sequence_length: int = 4096
    mask_token_id: int = 126336
    eos_token_id: int = 126081
    pad_token_id: int = 126081
    init_std: float = 0.02
    attention_dropout: float = 0.0
    residual_dropout: float = 0.0
    embedding_dropout: float = 0.0
    model_type: str = "llada"

    @property
    def effective_n_kv_heads(self) -> int:
        return self.n_kv_heads if self.n_kv_heads is not None else self.n_heads

    @property
    def ffn_size(self) -> int:
        return self.mlp_hidden_size if self.mlp_hidden_size is not None else self.mlp_ratio * self.d_model

    @classmethod
    def llada_8b(cls) -> "LLaDAConfig":
        return cls()


@dataclass
class DreamConfig:
    hidden_size: int = 3584
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    num_hidden_layers: int = 28
    intermediate_size: int = 18944
    hidden_act: str = "silu"
    vocab_size: int = 152064
    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 131072
    mask_token_id: int = 151666
    pad_token_id: int = 151643
    initializer_range: float = 0.02
    attention_dropout: float = 0.0
    model_type: str = "dream"

    @classmethod
    def dream_7b(cls) -> "DreamConfig":
        return cls()
