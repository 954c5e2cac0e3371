"""Model configuration.

``TransformerConfig`` carries the reference's fields (include/oil/transformer.h:12-25: vocab 32000,
hidden 768, 12 layers, 12 heads, head_dim 64, ffn 3072, eps 1e-5, rope theta 1e4, max_seq 2048, SiLU,
num_kv_heads with 0 meaning MHA, parallel residual) and adds what the reference fixes in code:
the norm kind, the position scheme, biases and MoE settings. ``pack_reference_struct`` /
``unpack_reference_struct`` convert to and from the 88-byte struct that the reference's
DenseModel::save writes into the ``.oil`` header (src/model.cpp:202-203).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field, asdict

ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2
_ACT_NAMES = {"relu": ACT_RELU, "gelu": ACT_GELU, "silu": ACT_SILU}


@dataclass
class TransformerConfig:
    vocab_size: int = 32000
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    head_dim: int = 64
    ffn_hidden_size: int = 3072
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq_len: int = 2048
    activation: str = "silu"          # "silu" => SwiGLU FFN (gate/up/down); "gelu"/"relu" => 2-layer FFN
    num_kv_heads: int = 0             # 0 = same as num_heads
    use_parallel_residual: bool = False
    # fields the reference hard-codes
    norm: str = "rmsnorm"             # "rmsnorm" | "layernorm"
    positions: str = "rope"           # "rope" | "learned"
    bias: bool = False
    tie_embeddings: bool = False
    # MoE (0 experts = dense)
    num_experts: int = 0
    top_k: int = 2
    moe_ffn_hidden_size: int = 0
    shared_expert: bool = False
    lb_coef: float = 0.01
    z_coef: float = 0.001
    # STE train-in-format quantisation of linear weights: "" | "oil8" | "oil4" | "spark" | "oil1"
    ste_format: str = ""
    ste_block: int = 32
    vocab_pad_to: int = 128
    gradient_checkpointing: bool = False

    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads if self.num_kv_heads > 0 else self.num_heads

    @property
    def padded_vocab(self) -> int:
        p = self.vocab_pad_to
        return (self.vocab_size + p - 1) // p * p

    def to_dict(self):
        return asdict(self)

    # ---- 88-byte reference struct: six i64, two f32, i64, u8 + 7 pad, i64, bool + 7 pad ----
    def pack_reference_struct(self) -> bytes:
        act = _ACT_NAMES.get(self.activation, ACT_SILU)
        return struct.pack("<6q2fqB7xqB7x", self.vocab_size, self.hidden_size, self.num_layers, self.num_heads, self.head_dim,
                           self.ffn_hidden_size, self.norm_eps, self.rope_theta, self.max_seq_len, act, self.num_kv_heads,
                           int(self.use_parallel_residual))

    @staticmethod
    def unpack_reference_struct(blob: bytes) -> "TransformerConfig":
        if len(blob) < 88:
            raise ValueError("config blob shorter than the 88-byte reference struct")
        v, hsz, nl, nh, hd, ffn, eps, theta, ms, act, nkv, par = struct.unpack("<6q2fqB7xqB7x", blob[:88])
        names = {v_: k for k, v_ in _ACT_NAMES.items()}
        return TransformerConfig(vocab_size=v, hidden_size=hsz, num_layers=nl, num_heads=nh, head_dim=hd, ffn_hidden_size=ffn,
                                 norm_eps=eps, rope_theta=theta, max_seq_len=ms, activation=names.get(act, "silu"), num_kv_heads=nkv,
                                 use_parallel_residual=bool(par))

    @staticmethod
    def unpack_packed(blob: bytes) -> "TransformerConfig":
        """The unpadded field order that InferenceEngine::deserialize_config reads
        (engines/inference/inference.cpp:45-70)."""
        v, hsz, nl, nh, hd, ffn, eps, theta, ms, act = struct.unpack("<6q2fqB", blob[:65])
        names = {v_: k for k, v_ in _ACT_NAMES.items()}
        nkv = struct.unpack("<q", blob[65:73])[0] if len(blob) >= 73 else 0
        return TransformerConfig(vocab_size=v, hidden_size=hsz, num_layers=nl, num_heads=nh, head_dim=hd, ffn_hidden_size=ffn,
                                 norm_eps=eps, rope_theta=theta, max_seq_len=ms, activation=names.get(act, "silu"), num_kv_heads=nkv)


def gpt2_small(**kw) -> TransformerConfig:
    """GPT-2-small-shaped decoder: 12 layers, d 768, 12 heads, FFN 3072 GELU, vocab 50257, context 1024."""
    base = dict(vocab_size=50257, hidden_size=768, num_layers=12, num_heads=12, head_dim=64, ffn_hidden_size=3072, max_seq_len=1024,
                activation="gelu", norm="layernorm", positions="learned", bias=True)
    base.update(kw)
    return TransformerConfig(**base)


def tiny_dense(**kw) -> TransformerConfig:
    """4 layers, d 256, 4 heads, FFN 1024 GELU, byte vocab, context 128, STE OIL8 block 32."""
    base = dict(vocab_size=256, hidden_size=256, num_layers=4, num_heads=4, head_dim=64, ffn_hidden_size=1024, max_seq_len=128,
                activation="gelu", norm="rmsnorm", positions="rope", bias=False, ste_format="oil8", ste_block=32, vocab_pad_to=1)
    base.update(kw)
    return TransformerConfig(**base)


def dense_64m(**kw) -> TransformerConfig:
    """The 14-layer, d 512 decoder (about 67 M weights, vocab 8192, context 2048) that the reference's train-in-format run and
    its speed probe use (tools/train_64m.cpp:63-71, tools/bench_speed.cpp:10-14)."""
    base = dict(vocab_size=8192, hidden_size=512, num_layers=14, num_heads=8, head_dim=64, ffn_hidden_size=2048, max_seq_len=2048,
                activation="silu", norm="rmsnorm", positions="rope", bias=False)
    base.update(kw)
    return TransformerConfig(**base)


def llama_7b(**kw) -> TransformerConfig:
    base = dict(vocab_size=32000, hidden_size=4096, num_layers=32, num_heads=32, head_dim=128, ffn_hidden_size=11008, max_seq_len=4096,
                activation="silu", num_kv_heads=8, norm="rmsnorm", positions="rope", bias=False)
    base.update(kw)
    return TransformerConfig(**base)


def dense_13b(**kw) -> TransformerConfig:
    base = dict(vocab_size=32000, hidden_size=5120, num_layers=40, num_heads=40, head_dim=128, ffn_hidden_size=13824, max_seq_len=4096,
                activation="silu", norm="rmsnorm", positions="rope", bias=False, ste_format="oil8", gradient_checkpointing=True)
    base.update(kw)
    return TransformerConfig(**base)


def moe_24l(**kw) -> TransformerConfig:
    base = dict(vocab_size=32000, hidden_size=2048, num_layers=24, num_heads=16, head_dim=128, ffn_hidden_size=5632, max_seq_len=2048,
                activation="silu", norm="rmsnorm", positions="rope", bias=False, num_experts=8, top_k=2, moe_ffn_hidden_size=5632)
    base.update(kw)
    return TransformerConfig(**base)


PRESETS = {"gpt2-small": gpt2_small, "tiny": tiny_dense, "dense-64m": dense_64m, "llama-7b": llama_7b, "dense-13b": dense_13b, "moe-24l": moe_24l}
