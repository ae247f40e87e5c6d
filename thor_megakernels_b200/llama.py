"""Llama model container: parameters, stacked weight views, KV cache, rotary
tables, and a plain PyTorch forward used for prefill.

The decode step itself runs in the CUDA megakernel; this module only owns the
tensors it reads and the host-side pieces around it.  Attribute paths follow the
reference's ``megakernels/llama.py`` so schedule builders and decode loops
written against it work unchanged:

* ``model.model.embed_tokens(BatchState)``            (reference :405-417)
* ``model.model.rope_cos`` / ``rope_sin`` fp32 tables  (reference :437-451)
* ``model.model.interleave_rope()``                    (reference :453-475)
* ``model.stack_params()`` -> ``model.stacked_params`` (reference :713-777)
* ``model.setup_caches()`` -> ``model.stacked_kv_cache`` ``[L,B,T,Hkv,D]`` (:552-574)
* ``model.lm_head.input_norm.weight`` / ``model.lm_head.lm_head.weight`` (:362-403)

Unlike the reference, no Hugging Face classes are needed: the config is a small
dataclass and the rotary tables (with the "llama3" frequency scaling) are
computed here.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .model_types import BatchState, DeviceType, ExtraModelConfig


@dataclass
class LlamaConfig:
    hidden_size: int = 2048
    num_hidden_layers: int = 16
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 64
    intermediate_size: int = 8192
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_position_embeddings: int = 131072
    tie_word_embeddings: bool = True
    rope_scaling: dict | None = field(
        default_factory=lambda: dict(
            rope_type="llama3",
            factor=32.0,
            low_freq_factor=1.0,
            high_freq_factor=4.0,
            original_max_position_embeddings=8192,
        )
    )


def config_from_pretrained(path) -> LlamaConfig:
    """``config.json`` of a Hugging Face Llama checkpoint directory -> ``LlamaConfig``
    (stands in for ``transformers.LlamaConfig.from_pretrained``, reference
    llama.py:596)."""
    import json
    from pathlib import Path

    raw = json.loads((Path(path) / "config.json").read_text())
    heads = raw["num_attention_heads"]
    scaling = raw.get("rope_scaling")
    if scaling is not None:
        scaling = dict(scaling)
        scaling.setdefault("rope_type", scaling.pop("type", "llama3"))
    return LlamaConfig(
        hidden_size=raw["hidden_size"], num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=heads,
        num_key_value_heads=raw.get("num_key_value_heads", heads), head_dim=raw.get("head_dim") or raw["hidden_size"] // heads,
        intermediate_size=raw["intermediate_size"], vocab_size=raw["vocab_size"], rms_norm_eps=raw.get("rms_norm_eps", 1e-5),
        rope_theta=raw.get("rope_theta", 500000.0), max_position_embeddings=raw.get("max_position_embeddings", 131072),
        tie_word_embeddings=raw.get("tie_word_embeddings", False), rope_scaling=scaling,
    )


def llama_1b_config(**overrides) -> LlamaConfig:
    """Llama-3.2-1B architecture."""
    return LlamaConfig(**overrides)


def llama_8b_config(**overrides) -> LlamaConfig:
    """Llama-3.1-8B architecture."""
    base = dict(
        hidden_size=4096,
        num_hidden_layers=32,
        num_attention_heads=32,
        num_key_value_heads=8,
        head_dim=128,
        intermediate_size=14336,
        vocab_size=128256,
        tie_word_embeddings=False,
        rope_scaling=dict(
            rope_type="llama3",
            factor=8.0,
            low_freq_factor=1.0,
            high_freq_factor=4.0,
            original_max_position_embeddings=8192,
        ),
    )
    base.update(overrides)
    return LlamaConfig(**base)


def rope_tables(cfg: LlamaConfig, num_positions: int | None = None) -> tuple[Tensor, Tensor]:
    """fp32 ``cos``/``sin`` tables ``[positions, head_dim]`` in the half-split
    ("rotate_half") column order: column ``i`` and ``i + D/2`` share frequency
    ``i``.  Frequencies follow the published Llama-3 rule: wavelengths longer
    than ``orig/low_freq_factor`` are divided by ``factor``, those shorter than
    ``orig/high_freq_factor`` are kept, and the band between is interpolated.
    """
    d = cfg.head_dim
    inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).to(torch.float32) / d))
    rs = cfg.rope_scaling
    if rs is not None and rs.get("rope_type", rs.get("type")) == "llama3":
        factor = rs["factor"]
        low, high = rs["low_freq_factor"], rs["high_freq_factor"]
        orig = rs["original_max_position_embeddings"]
        low_wavelen, high_wavelen = orig / low, orig / high
        wavelen = 2 * math.pi / inv_freq
        scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
        smooth = (orig / wavelen - low) / (high - low)
        blended = (1 - smooth) * scaled / factor + smooth * scaled
        in_band = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
        inv_freq = torch.where(in_band, blended, scaled)
    elif rs is not None:
        raise ValueError(f"unsupported rope_scaling {rs}")
    n = cfg.max_position_embeddings if num_positions is None else num_positions
    pos = torch.arange(n, dtype=torch.float32)
    freqs = (inv_freq[None, :, None] @ pos[None, None, :]).transpose(1, 2)[0]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half_interleaved(x: Tensor) -> Tensor:
    """(x0, x1, x2, x3, ...) -> (-x1, x0, -x3, x2, ...)."""
    return torch.stack((-x[..., 1::2], x[..., ::2]), dim=-1).view_as(x)


def rotate_half(x: Tensor) -> Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary_pos_emb_interleaved(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """Rotary embedding for the adjacent-pair layout (reference llama.py:149-174).
    bf16 inputs times fp32 tables promote to fp32; the caller rounds back."""
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    return (q * cos) + (rotate_half_interleaved(q) * sin), (k * cos) + (rotate_half_interleaved(k) * sin)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)


class RMSNorm(nn.Module):
    """fp32 normalisation, rounded to the input dtype, then scaled by the
    weight in that dtype (reference llama.py:29-47)."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.eps = cfg.rms_norm_eps
        self.weight = nn.Parameter(torch.ones(cfg.hidden_size))

    def forward(self, x: Tensor) -> Tensor:
        x32 = x.to(torch.float32)
        x32 = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * x32.to(x.dtype)


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig, extra: ExtraModelConfig, layer_idx: int):
        super().__init__()
        self.cfg, self.extra, self.layer_idx = cfg, extra, layer_idx
        self.input_layernorm = RMSNorm(cfg)
        d = cfg.head_dim
        self.q_proj = nn.Linear(cfg.hidden_size, cfg.num_attention_heads * d, bias=False)
        self.k_proj = nn.Linear(cfg.hidden_size, cfg.num_key_value_heads * d, bias=False)
        self.v_proj = nn.Linear(cfg.hidden_size, cfg.num_key_value_heads * d, bias=False)
        self.o_proj = nn.Linear(cfg.num_attention_heads * d, cfg.hidden_size, bias=False)
        self.kv_cache: tuple[Tensor, Tensor] | None = None

    def forward(self, state: BatchState) -> BatchState:
        cfg = self.cfg
        residual = state.hidden_states
        x = self.input_layernorm(residual)
        bsz, n = x.shape[:2]
        q = self.q_proj(x).view(bsz, n, cfg.num_attention_heads, -1)
        k = self.k_proj(x).view(bsz, n, cfg.num_key_value_heads, -1)
        v = self.v_proj(x).view(bsz, n, cfg.num_key_value_heads, -1)
        cos, sin = state.position_embeddings
        rope = apply_rotary_pos_emb_interleaved if self.extra.interleave_rope else apply_rotary_pos_emb
        dtype = q.dtype
        q, k = rope(q, k, cos, sin, unsqueeze_dim=-2)
        q, k = q.to(dtype), k.to(dtype)

        k_cache, v_cache = self.kv_cache
        k_cache[:, state.position_ids] = k
        v_cache[:, state.position_ids] = v
        if n > 1:  # prefill from position 0
            out = F.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True
            )
        else:
            out = F.scaled_dot_product_attention(
                q.transpose(1, 2),
                k_cache[:, : state.seq_len].transpose(1, 2),
                v_cache[:, : state.seq_len].transpose(1, 2),
                is_causal=False,
                enable_gqa=True,
            )
        out = out.transpose(1, 2).reshape(bsz, n, -1)
        state.hidden_states = residual + self.o_proj(out)
        return state


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, extra: ExtraModelConfig, layer_idx: int):
        super().__init__()
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)
        self.input_layernorm = RMSNorm(cfg)

    def forward(self, state: BatchState) -> BatchState:
        residual = state.hidden_states
        x = self.input_layernorm(residual)
        state.hidden_states = residual + self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))
        return state


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, extra: ExtraModelConfig, layer_idx: int):
        super().__init__()
        self.self_attn = LlamaAttention(cfg, extra, layer_idx)
        self.mlp = LlamaMLP(cfg, extra, layer_idx)

    def forward(self, state: BatchState) -> BatchState:
        return self.mlp(self.self_attn(state))


class LlamaLMHead(nn.Module):
    def __init__(self, cfg: LlamaConfig, extra: ExtraModelConfig):
        super().__init__()
        self.input_norm = RMSNorm(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)

    def forward(self, state: BatchState) -> BatchState:
        logits = self.lm_head(self.input_norm(state.hidden_states))
        state.output_ids = logits.argmax(dim=-1)
        return state


class LlamaEmbeddings(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)

    def forward(self, state: BatchState) -> BatchState:
        state.hidden_states = self.embed_tokens(state.input_ids)
        return state


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig, extra: ExtraModelConfig):
        super().__init__()
        self.config, self.extra_config = cfg, extra
        self.embed_tokens = LlamaEmbeddings(cfg)
        self.layers = nn.ModuleList(LlamaBlock(cfg, extra, i) for i in range(cfg.num_hidden_layers))
        n = extra.max_len_override or cfg.max_position_embeddings
        cos, sin = rope_tables(cfg, max(n, 1))
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def interleave_rope(self):
        """Switch to the adjacent-pair rotary layout the kernel uses: permute
        each head's Q/K output rows (and the table columns) from
        ``[0..D/2), [D/2..D)`` to ``0, D/2, 1, D/2+1, ...``.  Attention scores
        are unchanged because Q and K are permuted alike."""
        d = self.config.head_dim
        within = torch.stack((torch.arange(d // 2), torch.arange(d // 2) + d // 2), dim=-1).flatten()
        within = within.to(self.rope_cos.device)
        self.rope_cos = self.rope_cos[..., within].contiguous()
        self.rope_sin = self.rope_sin[..., within].contiguous()
        with torch.no_grad():
            for layer in self.layers:
                attn = layer.self_attn
                for proj, heads in ((attn.q_proj, self.config.num_attention_heads), (attn.k_proj, self.config.num_key_value_heads)):
                    rows = (torch.arange(heads, device=within.device)[:, None] * d + within[None, :]).flatten()
                    proj.weight[:] = proj.weight[rows.to(proj.weight.device)]

    def forward(self, state: BatchState) -> BatchState:
        state = self.embed_tokens(state)
        state.position_embeddings = (self.rope_cos[state.position_ids], self.rope_sin[state.position_ids])
        for layer in self.layers:
            state = layer(state)
        return state


@dataclass
class StackedParams:
    qkv_proj: Tensor
    o_proj: Tensor
    attn_ln_weight: Tensor
    mlp_ln_weight: Tensor
    up_proj: Tensor
    gate_proj: Tensor
    down_proj: Tensor


class LlamaForCausalLM(nn.Module):
    def __init__(self, config: LlamaConfig, extra_config: ExtraModelConfig | None = None):
        super().__init__()
        self.config = config
        self.extra_config = extra_config or ExtraModelConfig()
        self.device = torch.get_default_device()
        self.dtype = torch.get_default_dtype()
        self.model = LlamaModel(config, self.extra_config)
        self.lm_head = LlamaLMHead(config, self.extra_config)
        if config.tie_word_embeddings:
            self.lm_head.lm_head.weight = self.model.embed_tokens.embed_tokens.weight

    # -- construction ------------------------------------------------------
    @classmethod
    def random_init(
        cls,
        config: LlamaConfig,
        extra_config: ExtraModelConfig | None = None,
        seed: int = 0,
        std: float = 0.02,
        device: DeviceType = "cpu",
        dtype: torch.dtype = torch.bfloat16,
        generate_on: DeviceType = "cpu",
        finalize: bool = True,
    ) -> "LlamaForCausalLM":
        """Seeded random weights: every matrix ~ N(0, std) drawn in ``dtype`` in
        the order embedding, then per layer q, k, v, o, up, gate, down, then the
        LM head when it is not tied; norm weights are 1.  With
        ``generate_on="cpu"`` the result is identical on every machine; a CUDA
        ``generate_on`` draws from that device's generator instead (faster, but
        a different stream).  ``finalize=False`` returns the raw per-layer
        weights (Hugging Face row order) without stacking or cache allocation."""
        extra = extra_config or ExtraModelConfig(interleave_rope=True)
        prev = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            with torch.device("meta"):
                model = cls(config, extra)
        finally:
            torch.set_default_dtype(prev)
        gen_dev = torch.device(generate_on)
        gen = torch.Generator(device=gen_dev).manual_seed(seed)

        def draw(shape):
            return torch.empty(shape, dtype=dtype, device=gen_dev).normal_(0.0, std, generator=gen).to(device)

        def ones(shape):
            return torch.ones(shape, dtype=dtype, device=device)

        def put(param_owner, name, tensor):
            setattr(param_owner, name, nn.Parameter(tensor, requires_grad=False))

        emb = model.model.embed_tokens.embed_tokens
        put(emb, "weight", draw(emb.weight.shape))
        for layer in model.model.layers:
            attn, mlp = layer.self_attn, layer.mlp
            for lin in (attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj, mlp.up_proj, mlp.gate_proj, mlp.down_proj):
                put(lin, "weight", draw(lin.weight.shape))
            put(attn.input_layernorm, "weight", ones(attn.input_layernorm.weight.shape))
            put(mlp.input_layernorm, "weight", ones(mlp.input_layernorm.weight.shape))
        put(model.lm_head.input_norm, "weight", ones(model.lm_head.input_norm.weight.shape))
        if config.tie_word_embeddings:
            model.lm_head.lm_head.weight = emb.weight
        else:
            put(model.lm_head.lm_head, "weight", draw(model.lm_head.lm_head.weight.shape))

        n = extra.max_len_override or config.max_position_embeddings
        cos, sin = rope_tables(config, n)
        model.model.rope_cos = cos.to(device)
        model.model.rope_sin = sin.to(device)
        model.device, model.dtype = torch.device(device), dtype
        if finalize:
            model.finalize()
        return model

    # -- checkpoints -----------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_path, extra_config: ExtraModelConfig | None = None, device: DeviceType = "cpu",
                        dtype: torch.dtype = torch.bfloat16) -> "LlamaForCausalLM":
        """Load a Hugging Face Llama checkpoint directory (``config.json`` +
        safetensors) - reference llama.py:583-638.  With
        ``extra_config.tp_size > 1`` the model is built for rank
        ``extra_config.tp_rank``'s share - query and KV heads and the FFN width
        divided by ``tp_size`` (reference llama.py:192-207, 308-310) - and only
        that share of q/k/v/up/gate rows and o/down columns is read from disk
        (:665-691): the result has the layout ``tp.shard_model`` produces, except
        that embedding and LM head stay whole as in the reference.  Only local
        directories are supported (no download)."""
        import dataclasses
        from pathlib import Path

        extra = extra_config or ExtraModelConfig()
        path = Path(model_path)
        if not path.exists():
            raise FileNotFoundError(f"{model_path}: only local checkpoint directories can be loaded")
        cfg = config_from_pretrained(path)
        if extra.rope_scaling is not None:
            cfg = dataclasses.replace(cfg, rope_scaling=dict(extra.rope_scaling))
        whole = cfg
        if extra.tp_size > 1:
            for what, n in (("attention heads", cfg.num_attention_heads), ("KV heads", cfg.num_key_value_heads),
                            ("intermediate size", cfg.intermediate_size)):
                if n % extra.tp_size:
                    raise ValueError(f"{what} ({n}) do not divide over {extra.tp_size} ranks")
            cfg = dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // extra.tp_size,
                                      num_key_value_heads=cfg.num_key_value_heads // extra.tp_size,
                                      intermediate_size=cfg.intermediate_size // extra.tp_size)
        prev = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            with torch.device("meta"):
                model = cls(cfg, extra)
        finally:
            torch.set_default_dtype(prev)
        model.device, model.dtype = torch.device(device), dtype
        model.whole_config = whole
        model.load_from_safetensors(path)
        # rotary tables are buffers built on the meta device: rebuild them for real
        n = extra.max_len_override or cfg.max_position_embeddings
        cos, sin = rope_tables(cfg, max(n, 1))
        model.model.rope_cos, model.model.rope_sin = cos.to(device), sin.to(device)
        model.finalize()
        return model

    def make_name_to_hf_name(self) -> dict[str, str]:
        """This container's parameter names -> names in a Hugging Face Llama
        checkpoint (reference llama.py:640-663)."""
        names = {k: k for k in self.state_dict().keys()}
        for i in range(self.config.num_hidden_layers):
            names[f"model.layers.{i}.self_attn.input_layernorm.weight"] = f"model.layers.{i}.input_layernorm.weight"
            names[f"model.layers.{i}.mlp.input_layernorm.weight"] = f"model.layers.{i}.post_attention_layernorm.weight"
        names["model.embed_tokens.embed_tokens.weight"] = "model.embed_tokens.weight"
        names["lm_head.input_norm.weight"] = "model.norm.weight"
        names["lm_head.lm_head.weight"] = "model.embed_tokens.weight" if self.config.tie_word_embeddings else "lm_head.weight"
        return names

    def make_tp_map(self) -> dict[str, int]:
        """Hugging Face parameter name -> dimension it is split on across
        tensor-parallel ranks; parameters not listed are replicated (reference
        llama.py:665-691, keyed here by checkpoint name because that is what the
        loader sees)."""
        by_rows = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "up_proj.weight", "gate_proj.weight")
        by_cols = ("o_proj.weight", "down_proj.weight")
        out = {}
        for hf_name in self.make_name_to_hf_name().values():
            if hf_name.endswith(by_rows):
                out[hf_name] = 0
            elif hf_name.endswith(by_cols):
                out[hf_name] = 1
        return out

    def load_from_safetensors(self, model_path):
        """reference llama.py:693-711"""
        from .utils import load_safetensors_repo

        names = self.make_name_to_hf_name()
        hf = load_safetensors_repo(model_path, include_parameters=set(names.values()), device=self.device,
                                   tp_rank=self.extra_config.tp_rank, tp_size=self.extra_config.tp_size,
                                   tp_map=self.make_tp_map())
        state = {k: hf[v].to(self.dtype) for k, v in names.items()}
        self.load_state_dict(state, assign=True, strict=True)

    def to_hf_state_dict(self) -> dict[str, Tensor]:
        """Hugging Face-named tensors of a model that has NOT been finalised (row
        order as in a checkpoint); what ``save_file`` needs to write a checkpoint
        this class can load back."""
        state = self.state_dict()
        out = {}
        for name, hf_name in self.make_name_to_hf_name().items():
            out.setdefault(hf_name, state[name].detach().contiguous())
        return out

    def finalize(self):
        """What the reference's ``from_pretrained`` does after loading
        (llama.py:628-636): freeze, switch rotary layout, stack, allocate caches."""
        self.requires_grad_(False)
        if self.extra_config.interleave_rope:
            self.model.interleave_rope()
        self.stack_params()
        self.setup_caches()

    def to(self, device: DeviceType | None = None, dtype: torch.dtype | None = None):  # type: ignore[override]
        if device is not None:
            self.device = torch.device(device)
        if dtype is not None:
            self.dtype = dtype
        return super().to(device=device, dtype=dtype)

    # -- tensors the kernel reads ------------------------------------------
    def stack_params(self):
        """Layer-major stacked copies of every per-layer matrix; the per-layer
        modules are re-pointed at views of the stacks so both stay in sync."""
        layers = list(self.model.layers)

        def stack(mods):
            stacked = torch.stack([m.weight.data for m in mods], dim=0)
            for i, m in enumerate(mods):
                m.weight = nn.Parameter(stacked[i], requires_grad=False)
            return stacked

        cfg = self.config
        q_rows = cfg.num_attention_heads * cfg.head_dim
        kv_rows = cfg.num_key_value_heads * cfg.head_dim
        qkv = torch.stack(
            [torch.cat([l.self_attn.q_proj.weight.data, l.self_attn.k_proj.weight.data, l.self_attn.v_proj.weight.data], dim=0) for l in layers],
            dim=0,
        )
        for i, l in enumerate(layers):
            l.self_attn.q_proj.weight = nn.Parameter(qkv[i, :q_rows], requires_grad=False)
            l.self_attn.k_proj.weight = nn.Parameter(qkv[i, q_rows : q_rows + kv_rows], requires_grad=False)
            l.self_attn.v_proj.weight = nn.Parameter(qkv[i, q_rows + kv_rows :], requires_grad=False)

        self.stacked_params = StackedParams(
            qkv_proj=qkv,
            o_proj=stack([l.self_attn.o_proj for l in layers]),
            attn_ln_weight=stack([l.self_attn.input_layernorm for l in layers]),
            mlp_ln_weight=stack([l.mlp.input_layernorm for l in layers]),
            up_proj=stack([l.mlp.up_proj for l in layers]),
            gate_proj=stack([l.mlp.gate_proj for l in layers]),
            down_proj=stack([l.mlp.down_proj for l in layers]),
        )

    def setup_caches(self):
        cfg, extra = self.config, self.extra_config
        shape = (
            cfg.num_hidden_layers,
            extra.max_batch_size,
            extra.max_len_override or cfg.max_position_embeddings,
            cfg.num_key_value_heads,
            cfg.head_dim,
        )
        k = torch.zeros(shape, device=self.device, dtype=self.dtype)
        v = torch.zeros(shape, device=self.device, dtype=self.dtype)
        self.stacked_kv_cache = (k, v)
        for i, layer in enumerate(self.model.layers):
            layer.self_attn.kv_cache = (k[i], v[i])

    # -- plain PyTorch forward (prefill) -----------------------------------
    @torch.no_grad()
    def forward(self, batch_state: BatchState) -> BatchState:
        ids, pos = batch_state.input_ids, batch_state.position_ids
        ids = ids.unsqueeze(0) if ids.ndim == 1 else ids
        pos = pos.unsqueeze(0) if pos.ndim == 1 else pos
        state = BatchState(input_ids=ids, position_ids=pos, hidden_states=batch_state.hidden_states, seq_len=batch_state.seq_len)
        return self.lm_head(self.model(state))
