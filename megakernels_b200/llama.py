"""Llama model container for the decode megakernel.

This is not a torch ``nn.Module`` forward implementation: the decode forward
pass runs entirely inside the CUDA megakernel.  The container only owns what
the kernel's globals are built from (reference: megakernels/llama.py):

* the embedding table and ``embed_tokens`` lookup        (llama.py:406-417)
* per-layer weights stacked over layers, q/k/v fused      (llama.py:713-777)
* the stacked KV cache ``[L, B, T, Hkv, D]``              (llama.py:552-574)
* fp32 RoPE cos/sin tables, optionally interleaved        (llama.py:440-475)
* the final norm weight and LM-head weight                (llama.py:369-403)

Weights come either from a seeded random initialisation (the benchmark
configurations are random-init by definition) or from a directory of
``safetensors`` files in Hugging Face layout.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch
from torch import Tensor

from megakernels_b200.model_types import BatchState, DeviceType, ExtraModelConfig


# --------------------------------------------------------------------------- #
# configuration
# --------------------------------------------------------------------------- #

LLAMA3_ROPE_SCALING = dict(
    factor=32.0,
    low_freq_factor=1.0,
    high_freq_factor=4.0,
    original_max_position_embeddings=8192,
    rope_type="llama3",
)


@dataclass
class LlamaConfig:
    """The subset of the Hugging Face Llama config the decode path needs."""

    hidden_size: int = 2048
    intermediate_size: int = 8192
    num_hidden_layers: int = 16
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 64
    vocab_size: int = 128256
    max_position_embeddings: int = 131072
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    tie_word_embeddings: bool = True
    rope_scaling: dict | None = field(default_factory=lambda: dict(LLAMA3_ROPE_SCALING))

    @classmethod
    def llama_3_2_1b(cls, **overrides) -> "LlamaConfig":
        return cls(**overrides)

    @classmethod
    def llama_3_1_8b(cls, **overrides) -> "LlamaConfig":
        base = dict(
            hidden_size=4096,
            intermediate_size=14336,
            num_hidden_layers=32,
            num_attention_heads=32,
            num_key_value_heads=8,
            head_dim=128,
            tie_word_embeddings=False,
            rope_scaling=dict(LLAMA3_ROPE_SCALING, factor=8.0),
        )
        base.update(overrides)
        return cls(**base)

    @classmethod
    def llama_3_1_70b(cls, **overrides) -> "LlamaConfig":
        base = dict(
            hidden_size=8192,
            intermediate_size=28672,
            num_hidden_layers=80,
            num_attention_heads=64,
            num_key_value_heads=8,
            head_dim=128,
            tie_word_embeddings=False,
            rope_scaling=dict(LLAMA3_ROPE_SCALING, factor=8.0),
        )
        base.update(overrides)
        return cls(**base)

    @classmethod
    def from_json(cls, path: Path) -> "LlamaConfig":
        raw = json.loads(Path(path).read_text())
        head_dim = raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"]
        return cls(
            hidden_size=raw["hidden_size"],
            intermediate_size=raw["intermediate_size"],
            num_hidden_layers=raw["num_hidden_layers"],
            num_attention_heads=raw["num_attention_heads"],
            num_key_value_heads=raw["num_key_value_heads"],
            head_dim=head_dim,
            vocab_size=raw["vocab_size"],
            max_position_embeddings=raw["max_position_embeddings"],
            rms_norm_eps=raw["rms_norm_eps"],
            rope_theta=raw.get("rope_theta", 10000.0),
            tie_word_embeddings=raw.get("tie_word_embeddings", False),
            rope_scaling=raw.get("rope_scaling"),
        )


# --------------------------------------------------------------------------- #
# rotary tables
# --------------------------------------------------------------------------- #


def rope_inverse_frequencies(config: LlamaConfig) -> Tensor:
    """fp32 inverse frequencies with the published Llama-3 wavelength scaling.

    The reference obtains these from ``transformers``' ``LlamaRotaryEmbedding``
    (megakernels/llama.py:436-451); the arithmetic is restated here so the
    product does not depend on ``transformers``.
    """
    dim = config.head_dim
    inv_freq = 1.0 / (
        config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim)
    )
    sc = config.rope_scaling
    if not sc or sc.get("rope_type", sc.get("type", "default")) == "default":
        return inv_freq
    kind = sc.get("rope_type", sc.get("type"))
    if kind != "llama3":
        raise ValueError(f"unsupported rope scaling {kind!r}")
    factor = sc["factor"]
    low = sc["low_freq_factor"]
    high = sc["high_freq_factor"]
    old_len = sc["original_max_position_embeddings"]
    low_wavelen = old_len / low
    high_wavelen = old_len / high
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old_len / wavelen - low) / (high - low)
    blended = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) * ~(wavelen > low_wavelen)
    return torch.where(medium, blended, scaled)


def build_rope_tables(config: LlamaConfig, num_positions: int, interleave: bool):
    """cos/sin tables ``[num_positions, head_dim]`` in fp32.

    Non-interleaved layout is ``cat(freqs, freqs)``; the interleaved layout
    repeats each frequency on adjacent columns ``(2i, 2i+1)``, which is what
    the column permutation of megakernels/llama.py:453-465 produces.
    """
    inv_freq = rope_inverse_frequencies(config)
    pos = torch.arange(num_positions, dtype=torch.float32)
    freqs = (inv_freq[:, None].float() @ pos[None, :].float()).transpose(0, 1)
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos(), emb.sin()
    if interleave:
        idx = interleave_indices(config.head_dim, 1)
        cos, sin = cos[:, idx], sin[:, idx]
    return cos.contiguous(), sin.contiguous()


def interleave_indices(head_dim: int, num_heads: int) -> Tensor:
    """Row permutation that makes RoPE pairs ``(i, i + D/2)`` adjacent.

    Reference: megakernels/llama.py:453-475 (``interleave_rope``).
    """
    half = head_dim // 2
    one = torch.stack((torch.arange(half), torch.arange(half) + half), dim=1).reshape(-1)
    return (one[None, :] + head_dim * torch.arange(num_heads)[:, None]).reshape(-1)


# --------------------------------------------------------------------------- #
# parameter containers
# --------------------------------------------------------------------------- #


@dataclass
class StackedParams:
    """Reference: megakernels/llama.py:478-486."""

    qkv_proj: Tensor
    o_proj: Tensor
    attn_ln_weight: Tensor
    mlp_ln_weight: Tensor
    up_proj: Tensor
    gate_proj: Tensor
    down_proj: Tensor


class _Weight:
    def __init__(self, weight: Tensor):
        self.weight = weight


class LlamaEmbeddings:
    """Token embedding lookup (reference: megakernels/llama.py:406-417)."""

    def __init__(self, weight: Tensor):
        self.embed_tokens = _Weight(weight)

    def __call__(self, batch_state: BatchState) -> BatchState:
        batch_state.hidden_states = self.embed_tokens.weight[batch_state.input_ids]
        return batch_state


class LlamaLMHead:
    """Holds the final norm and LM-head weights (llama.py:369-403)."""

    def __init__(self, norm_weight: Tensor, head_weight: Tensor):
        self.input_norm = _Weight(norm_weight)
        self.lm_head = _Weight(head_weight)


class LlamaModel:
    def __init__(self, embed: LlamaEmbeddings, rope_cos: Tensor, rope_sin: Tensor):
        self.embed_tokens = embed
        self.rope_cos = rope_cos
        self.rope_sin = rope_sin


def compute_shard_bounds(dim_size: int, num_shards: int, shard_index: int) -> slice:
    """Reference: megakernels/utils.py:16-31."""
    base, rem = divmod(dim_size, num_shards)
    start = shard_index * base + min(shard_index, rem)
    return slice(start, start + base + (1 if shard_index < rem else 0))


class LlamaForCausalLM:
    """Weights, KV cache and RoPE tables in the layout the megakernel reads."""

    def __init__(
        self,
        config: LlamaConfig,
        extra_config: ExtraModelConfig,
        device: DeviceType,
        dtype: torch.dtype,
        embed_weight: Tensor,
        stacked: StackedParams,
        final_norm_weight: Tensor,
        lm_head_weight: Tensor,
    ):
        self.config = config
        self.extra_config = extra_config
        self.device = torch.device(device)
        self.dtype = dtype
        self.stacked_params = stacked
        self.lm_head = LlamaLMHead(final_norm_weight, lm_head_weight)
        n_pos = self.kv_len()
        cos, sin = build_rope_tables(config, n_pos, extra_config.interleave_rope)
        self.model = LlamaModel(
            LlamaEmbeddings(embed_weight), cos.to(self.device), sin.to(self.device)
        )
        self.setup_caches()

    # -- geometry --------------------------------------------------------- #
    def kv_len(self) -> int:
        return self.extra_config.max_len_override or self.config.max_position_embeddings

    def num_kv_heads(self) -> int:
        tp = self.extra_config.tp_size
        assert self.config.num_key_value_heads % tp == 0
        return self.config.num_key_value_heads // tp

    def num_qo_heads(self) -> int:
        tp = self.extra_config.tp_size
        assert self.config.num_attention_heads % tp == 0
        return self.config.num_attention_heads // tp

    def local_intermediate_size(self) -> int:
        tp = self.extra_config.tp_size
        assert self.config.intermediate_size % tp == 0
        return self.config.intermediate_size // tp

    def setup_caches(self) -> None:
        """Zeroed stacked KV cache (reference: megakernels/llama.py:552-574)."""
        shape = (
            self.config.num_hidden_layers,
            self.extra_config.max_batch_size,
            self.kv_len(),
            self.num_kv_heads(),
            self.config.head_dim,
        )
        k_cache = torch.zeros(shape, device=self.device, dtype=self.dtype)
        self.stacked_kv_cache = (k_cache, torch.zeros_like(k_cache))

    # -- construction ----------------------------------------------------- #
    @classmethod
    def from_random(
        cls,
        config: LlamaConfig,
        extra_config: ExtraModelConfig | None = None,
        device: DeviceType = "cuda:0",
        dtype: torch.dtype = torch.bfloat16,
        seed: int = 0,
        std: float = 0.02,
        draw_on: str = "cpu",
    ) -> "LlamaForCausalLM":
        """Seeded ``N(0, std)`` matrices, RMSNorm weights 1.0.

        With ``draw_on="cpu"`` every matrix is drawn in fp32 from one CPU
        generator in the parameter order of the reference model (embedding;
        per layer q, k, v, o, up, gate, down; then the untied LM head), cast to
        ``dtype``, and only then sharded, so all tensor-parallel ranks hold
        slices of the same tensors and a CPU reference built from the same seed
        sees identical values.  ``draw_on="device"`` draws each matrix directly
        on the target device (same distribution, different values); it exists
        for full-size benchmark models where a CPU draw would take minutes.
        """
        extra = extra_config or ExtraModelConfig()
        device = torch.device(device)
        H, I, L = config.hidden_size, config.intermediate_size, config.num_hidden_layers
        D, Hq, Hkv, V = (
            config.head_dim,
            config.num_attention_heads,
            config.num_key_value_heads,
            config.vocab_size,
        )
        tp, rank = extra.tp_size, extra.tp_rank

        if draw_on == "cpu":
            gen = torch.Generator().manual_seed(seed)

            def draw(*shape):
                w = torch.randn(shape, generator=gen, dtype=torch.float32) * std
                return w.to(dtype)

        elif draw_on == "device":
            gen = torch.Generator(device=device).manual_seed(seed)

            def draw(*shape):
                w = torch.empty(shape, device=device, dtype=dtype)
                # chunked so the fp32 temporary stays small next to a 180 GB HBM
                rows = max(1, (1 << 28) // max(1, shape[-1]))
                for r0 in range(0, shape[0], rows):
                    r1 = min(shape[0], r0 + rows)
                    tmp = torch.randn(
                        (r1 - r0, *shape[1:]), generator=gen, device=device, dtype=torch.float32
                    )
                    w[r0:r1] = (tmp * std).to(dtype)
                return w

        elif draw_on == "zeros":
            # shape-only model (schedules, argument marshalling): no values drawn
            def draw(*shape):
                return torch.zeros(shape, dtype=dtype, device=device)

        else:
            raise ValueError(f"draw_on must be 'cpu', 'device' or 'zeros', not {draw_on!r}")

        q_perm = interleave_indices(D, Hq) if extra.interleave_rope else None
        k_perm = interleave_indices(D, Hkv) if extra.interleave_rope else None

        def rows(w: Tensor, n_units: int) -> Tensor:
            # split the output rows into ``n_units`` equal units and keep this rank's
            unit = w.shape[0] // n_units
            sl = compute_shard_bounds(n_units, tp, rank)
            return w[sl.start * unit : sl.stop * unit]

        def cols(w: Tensor, n_units: int) -> Tensor:
            unit = w.shape[1] // n_units
            sl = compute_shard_bounds(n_units, tp, rank)
            return w[:, sl.start * unit : sl.stop * unit]

        embed = draw(V, H).to(device)
        qkv, o, up, gate, down = [], [], [], [], []
        for _ in range(L):
            q = draw(Hq * D, H)
            k = draw(Hkv * D, H)
            v = draw(Hkv * D, H)
            if q_perm is not None:
                q = q[q_perm.to(q.device)]
                k = k[k_perm.to(k.device)]
            qkv.append(torch.cat([rows(q, Hq), rows(k, Hkv), rows(v, Hkv)], dim=0).to(device))
            o.append(cols(draw(H, Hq * D), Hq).contiguous().to(device))
            up.append(rows(draw(I, H), tp).to(device))
            gate.append(rows(draw(I, H), tp).to(device))
            down.append(cols(draw(H, I), tp).contiguous().to(device))
        head = embed if config.tie_word_embeddings else draw(V, H).to(device)

        stacked = StackedParams(
            qkv_proj=torch.stack(qkv),
            o_proj=torch.stack(o),
            attn_ln_weight=torch.ones(L, H, device=device, dtype=dtype),
            mlp_ln_weight=torch.ones(L, H, device=device, dtype=dtype),
            up_proj=torch.stack(up),
            gate_proj=torch.stack(gate),
            down_proj=torch.stack(down),
        )
        del qkv, o, up, gate, down
        return cls(
            config,
            extra,
            device,
            dtype,
            embed,
            stacked,
            torch.ones(H, device=device, dtype=dtype),
            head,
        )

    @classmethod
    def from_pretrained(
        cls,
        model_path: str | Path,
        extra_config: ExtraModelConfig | None = None,
        device: DeviceType = "cuda:0",
        dtype: torch.dtype = torch.bfloat16,
    ) -> "LlamaForCausalLM":
        """Load a local Hugging Face checkpoint directory (``*.safetensors``).

        Reference: megakernels/llama.py:583-711 and utils.py:34-97 (name map,
        shard-on-load).  Only local directories are supported.
        """
        from safetensors import safe_open

        extra = extra_config or ExtraModelConfig()
        path = Path(model_path)
        config = LlamaConfig.from_json(path / "config.json")
        if extra.rope_scaling is not None:
            config.rope_scaling = extra.rope_scaling
        files = sorted(path.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no safetensors files under {path}")
        where: dict[str, Path] = {}
        for f in files:
            with safe_open(f, framework="pt", device="cpu") as fh:
                for k in fh.keys():
                    where[k] = f

        def get(name: str) -> Tensor:
            with safe_open(where[name], framework="pt", device="cpu") as fh:
                return fh.get_tensor(name).to(dtype)

        tp, rank = extra.tp_size, extra.tp_rank
        D, Hq, Hkv = config.head_dim, config.num_attention_heads, config.num_key_value_heads
        q_perm = interleave_indices(D, Hq) if extra.interleave_rope else None
        k_perm = interleave_indices(D, Hkv) if extra.interleave_rope else None

        def rows(w, n_units):
            unit = w.shape[0] // n_units
            sl = compute_shard_bounds(n_units, tp, rank)
            return w[sl.start * unit : sl.stop * unit]

        def cols(w, n_units):
            unit = w.shape[1] // n_units
            sl = compute_shard_bounds(n_units, tp, rank)
            return w[:, sl.start * unit : sl.stop * unit]

        device = torch.device(device)
        embed = get("model.embed_tokens.weight").to(device)
        qkv, o, up, gate, down, ln1, ln2 = [], [], [], [], [], [], []
        for i in range(config.num_hidden_layers):
            p = f"model.layers.{i}."
            q, k, v = (get(p + f"self_attn.{n}_proj.weight") for n in "qkv")
            if q_perm is not None:
                q, k = q[q_perm], k[k_perm]
            qkv.append(torch.cat([rows(q, Hq), rows(k, Hkv), rows(v, Hkv)]).to(device))
            o.append(cols(get(p + "self_attn.o_proj.weight"), Hq).contiguous().to(device))
            up.append(rows(get(p + "mlp.up_proj.weight"), tp).to(device))
            gate.append(rows(get(p + "mlp.gate_proj.weight"), tp).to(device))
            down.append(cols(get(p + "mlp.down_proj.weight"), tp).contiguous().to(device))
            ln1.append(get(p + "input_layernorm.weight").to(device))
            ln2.append(get(p + "post_attention_layernorm.weight").to(device))
        head = embed if config.tie_word_embeddings else get("lm_head.weight").to(device)
        stacked = StackedParams(
            qkv_proj=torch.stack(qkv),
            o_proj=torch.stack(o),
            attn_ln_weight=torch.stack(ln1),
            mlp_ln_weight=torch.stack(ln2),
            up_proj=torch.stack(up),
            gate_proj=torch.stack(gate),
            down_proj=torch.stack(down),
        )
        return cls(
            config, extra, device, dtype, embed, stacked, get("model.norm.weight").to(device), head
        )
