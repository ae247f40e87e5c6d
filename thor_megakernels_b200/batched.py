"""Batched-decode operators (16..128 sequences per step) on the tcgen05 tensor
cores, through the C-ABI library.

``linear`` is the dense contraction every linear layer becomes once a decode
step carries a batch: ``y[b, n] = sum_k x[b, k] * W[n, k]``.  The reference's
operator of this shape is ``include/ops/nvfp4_linear.cuh:52-173``.
"""
from __future__ import annotations

import torch

from . import _lib


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


_error_words: dict = {}


def _error_word(device: torch.device) -> torch.Tensor:
    word = _error_words.get(device.index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _error_words[device.index] = word
    return word


def suggested_splits(n: int, k: int, device=None) -> int:
    sms = torch.cuda.get_device_properties(device or torch.cuda.current_device()).multi_processor_count
    return int(_lib.load().mk_linear_batched_splits(n, k, sms))


def linear(weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None, splits: int = 1,
           partials: torch.Tensor | None = None) -> torch.Tensor:
    """``weight`` bf16 ``[n, k]``, ``x`` bf16 ``[batch <= 128, k]``; returns bf16
    ``[batch, n]`` (fp32 accumulation, one rounding).  With ``splits > 1`` the K
    dimension is divided over several CTAs per 128-row slab and the fp32 partial
    sums ``[splits, batch, n]`` are returned instead, to be added in split order
    by the caller."""
    for name, t in (("weight", weight), ("x", x)):
        if t.device.type != "cuda" or t.dtype != torch.bfloat16 or not t.is_contiguous() or t.ndim != 2:
            raise ValueError(f"{name} must be a contiguous 2-D bf16 CUDA tensor")
    n, k = weight.shape
    batch = x.shape[0]
    if x.shape[1] != k:
        raise ValueError(f"x has {x.shape[1]} columns, weight has {k}")
    lib = _lib.load()
    err = _error_word(x.device)
    if splits == 1:
        y = out if out is not None else torch.empty((batch, n), dtype=torch.bfloat16, device=x.device)
        part_ptr = None
    else:
        y = None
        if partials is None:
            partials = torch.empty((splits, batch, n), dtype=torch.float32, device=x.device)
        part_ptr = partials.data_ptr()
    with torch.cuda.device(x.device):
        _lib.check(lib.mk_linear_batched(weight.data_ptr(), x.data_ptr(), None if y is None else y.data_ptr(), part_ptr,
                                         n, k, batch, splits, err.data_ptr(), _stream(x)))
    return y if splits == 1 else partials


class Nvfp4Native:
    """A matrix quantised to NVFP4 with its block scales in the tensor core's
    native layout (``mk_nvfp4_quantize_native``)."""

    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, tensor_scale: float, rows: int, k: int):
        self.packed, self.scales, self.tensor_scale, self.rows, self.k = packed, scales, float(tensor_scale), rows, k

    def canonical_scales(self) -> torch.Tensor:
        """The scale bytes as a row-major ``[rows, k/16]`` matrix (the layout of
        the weight-only path and of the reference's ``canonical`` output)."""
        groups = self.k // 16
        atoms = self.scales.view((self.rows + 127) // 128, groups // 4, 32, 4, 4)   # [slab, g/4, r%32, r%128//32, g%4]
        rows = atoms.permute(0, 3, 2, 1, 4).reshape(-1, groups)                     # [slab, quarter, r%32] -> row ; [g/4, g%4] -> g
        return rows[: self.rows].contiguous()


def quantize_native(x: torch.Tensor, tensor_scale: float | None = None) -> Nvfp4Native:
    """bf16 ``[rows, k]`` (k a multiple of 64) -> NVFP4 codes + native-layout
    block scales.  ``tensor_scale`` defaults to ``amax / (6 * 448)`` as for weights."""
    if x.device.type != "cuda" or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.ndim != 2:
        raise ValueError("x must be a contiguous 2-D bf16 CUDA tensor")
    rows, k = x.shape
    lib = _lib.load()
    if tensor_scale is None:
        from .nvfp4 import tensor_scale_for

        tensor_scale = tensor_scale_for(x)
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.zeros(max(1, int(lib.mk_nvfp4_native_scale_bytes(rows, k))), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.mk_nvfp4_quantize_native(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), rows, k, float(tensor_scale),
                                                _stream(x)))
    return Nvfp4Native(packed, scales, tensor_scale, rows, k)


def linear_nvfp4(weight: Nvfp4Native, x: Nvfp4Native, out: torch.Tensor | None = None) -> torch.Tensor:
    """``y[b, n] = bf16(ts_w * ts_x * sum_k w[n, k] x[b, k])`` with both operands in
    NVFP4, the block scales applied by the tensor core."""
    if weight.k != x.k:
        raise ValueError(f"x has {x.k} columns, weight has {weight.k}")
    lib = _lib.load()
    dev = x.packed.device
    y = out if out is not None else torch.empty((x.rows, weight.rows), dtype=torch.bfloat16, device=dev)
    err = _error_word(dev)
    with torch.cuda.device(dev):
        _lib.check(lib.mk_linear_batched_nvfp4(weight.packed.data_ptr(), weight.scales.data_ptr(), weight.tensor_scale,
                                               x.packed.data_ptr(), x.scales.data_ptr(), x.tensor_scale, y.data_ptr(), None,
                                               weight.rows, weight.k, x.rows, 1, err.data_ptr(),
                                               torch.cuda.current_stream(dev).cuda_stream))
    return y


class BatchedDecoder:
    """Greedy decode of up to 128 sequences per step, each with its own cache
    length (``mk_batched_create`` / ``mk_step_batched``).

    ``model`` is a finalised model container whose caches were set up with
    ``ExtraModelConfig(max_batch_size >= max_batch)``; sequence ``b`` lives in
    cache slot ``b``.  After ``step`` the residual stream is in ``hidden``
    ``[batch, hidden]`` and the logits in ``logits`` ``[batch, vocab]``."""

    def __init__(self, model, max_batch: int, quantized: dict | None = None, activation_scale: float = 1.0):
        """``quantized``: result of ``nvfp4.quantize_model(model)`` to run every
        linear as NVFP4 x NVFP4 on the block-scaled tensor-core path (the
        activations are quantised on the fly with ``activation_scale`` as their
        tensor scale); default: bf16 weights."""
        import ctypes as C
        import math

        cfg = model.config
        dev = model.device
        sp = model.stacked_params
        k, v = model.stacked_kv_cache
        self.device = torch.device(dev)
        self.max_batch = max_batch
        self.hidden = torch.zeros((max_batch, cfg.hidden_size), dtype=torch.bfloat16, device=dev)
        self.logits = torch.zeros((max_batch, cfg.vocab_size), dtype=torch.bfloat16, device=dev)
        embed = model.model.embed_tokens.embed_tokens.weight.data
        head = model.lm_head.lm_head.weight.data
        self._keep = [sp, k, v, embed, head, model.model.rope_cos, model.model.rope_sin, model.lm_head.input_norm.weight]
        d = _lib.MkModelDesc()
        d.abi_version = _lib.MK_ABI_VERSION
        d.weight_format = _lib.MK_WEIGHTS_BF16 if quantized is None else _lib.MK_WEIGHTS_NVFP4
        d.hidden_size, d.num_layers = cfg.hidden_size, cfg.num_hidden_layers
        d.num_q_heads, d.num_kv_heads, d.head_dim = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        d.intermediate_size, d.vocab_size = cfg.intermediate_size, cfg.vocab_size
        d.attn_scale, d.rms_norm_eps = 1 / math.sqrt(cfg.head_dim), float(cfg.rms_norm_eps)
        if quantized is None:
            d.qkv_w, d.o_w, d.up_w = sp.qkv_proj.data_ptr(), sp.o_proj.data_ptr(), sp.up_proj.data_ptr()
            d.gate_w, d.down_w, d.lm_head_w = sp.gate_proj.data_ptr(), sp.down_proj.data_ptr(), head.data_ptr()
        else:
            self._tables = {}
            for key, field in (("qkv", "qkv_q"), ("o", "o_q"), ("up", "up_q"), ("gate", "gate_q"), ("down", "down_q"),
                               ("lm_head", "lm_head_q")):
                mats = quantized[key] if key != "lm_head" else [quantized[key]]
                table = (_lib.MkNvfp4Matrix * len(mats))()
                for i, m in enumerate(mats):
                    table[i].packed, table[i].scales = m.packed.data_ptr(), m.scales.data_ptr()
                    table[i].tensor_scale = float(m.tensor_scale)
                self._tables[key] = (table, mats)
                setattr(d, field, table)
        d.attn_norm_w, d.mlp_norm_w = sp.attn_ln_weight.data_ptr(), sp.mlp_ln_weight.data_ptr()
        d.lm_head_norm_w, d.embed_w = model.lm_head.input_norm.weight.data_ptr(), embed.data_ptr()
        d.k_cache, d.v_cache, d.kv_batch, d.kv_max_len = k.data_ptr(), v.data_ptr(), k.shape[1], k.shape[2]
        d.rope_cos, d.rope_sin = model.model.rope_cos.data_ptr(), model.model.rope_sin.data_ptr()
        d.rope_positions = model.model.rope_cos.shape[0]
        d.hidden_states, d.logits = self.hidden.data_ptr(), self.logits.data_ptr()
        self.kv_max_len, self.kv_batch = k.shape[2], k.shape[1]
        self.lib = _lib.load()
        self.handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_batched_create(C.byref(d), max_batch, C.byref(self.handle)))
            if quantized is not None:
                _lib.check(self.lib.mk_batched_set_activation_scale(self.handle, float(activation_scale)))

    def step(self, tokens: torch.Tensor, pos_ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``tokens`` and ``pos_ids``: int32 CUDA vectors of the same length
        (``<= max_batch``).  Returns the greedy tokens (int32)."""
        for name, t in (("tokens", tokens), ("pos_ids", pos_ids)):
            if t.device.type != "cuda" or t.dtype != torch.int32 or t.ndim != 1 or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous int32 CUDA vector")
        batch = tokens.numel()
        if pos_ids.numel() != batch:
            raise ValueError("tokens and pos_ids differ in length")
        if batch > self.kv_batch:
            raise ValueError(f"the model's cache holds {self.kv_batch} sequences, the batch has {batch}")
        if out is None:
            out = torch.empty(batch, dtype=torch.int32, device=tokens.device)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_step_batched(self.handle, tokens.data_ptr(), pos_ids.data_ptr(), batch, out.data_ptr(),
                                                _stream(tokens)))
        return out

    def prefill(self, tokens: torch.Tensor, slot: int = 0, start_pos: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
        """Process a prompt on the device (replaces the PyTorch forward the
        reference uses for prefill): ``tokens`` (int32 CUDA vector) go to positions
        ``start_pos ..`` of cache slot ``slot``.  Returns a 1-element int32 tensor
        with the greedy token that follows the prompt; ``logits[0]`` are its logits."""
        if tokens.device.type != "cuda" or tokens.dtype != torch.int32 or tokens.ndim != 1 or not tokens.is_contiguous():
            raise ValueError("tokens must be a contiguous int32 CUDA vector")
        if out is None:
            out = torch.empty(1, dtype=torch.int32, device=tokens.device)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_prefill_batched(self.handle, tokens.data_ptr(), tokens.numel(), int(slot), int(start_pos),
                                                   out.data_ptr(), _stream(tokens)))
        return out

    def status(self):
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_batched_status(self.handle, torch.cuda.current_stream(self.device).cuda_stream))

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.mk_batched_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def check_errors(device=None) -> None:
    """Synchronises and raises if a bounded wait inside a batched kernel ran out."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    torch.cuda.synchronize(device)
    word = _error_words.get(device.index)
    if word is not None and int(word.item()) != 0:
        word.zero_()
        raise _lib.MegakernelError(_lib.MK_ERR_DEVICE_WAIT, "a bounded wait inside a batched-decode kernel ran out")


class ThroughputExecutor:
    """The reference's batched instruction set (``demos/throughput``) on the
    tensor-core batched path: binds a ``Globals``' tensors once, validates an
    instruction tensor (``set_schedule``) and runs the operators it covers for
    one decode step at a single ``pos_id`` (``step``).  Semantics follow the
    reference's interpreter (``megakernels/demos/throughput/python_vm.py``):
    half-split rotary embedding, residual stream in and out through
    ``hidden_states``, counters left at their final values in ``barriers``."""

    def __init__(self, *, barriers, qkv_w, attn_norm_w, o_w, mlp_norm_w, up_w, gate_w, down_w, lm_head_norm_w, lm_head_w,
                 k_cache, v_cache, rope_cos, rope_sin, hidden_states, rms_rope_intermediates, rms_gate_intermediates,
                 post_ln_rope_q, attn_out, silu_out, rms_lm_head_intermediates, logits, attn_scale, rms_norm_eps, batch_size):
        import ctypes as C

        tensors = dict(barriers=barriers, qkv_w=qkv_w, attn_norm_w=attn_norm_w, o_w=o_w, mlp_norm_w=mlp_norm_w, up_w=up_w,
                       gate_w=gate_w, down_w=down_w, lm_head_norm_w=lm_head_norm_w, lm_head_w=lm_head_w, k_cache=k_cache,
                       v_cache=v_cache, rope_cos=rope_cos, rope_sin=rope_sin, hidden_states=hidden_states,
                       rms_rope_intermediates=rms_rope_intermediates, rms_gate_intermediates=rms_gate_intermediates,
                       post_ln_rope_q=post_ln_rope_q, attn_out=attn_out, silu_out=silu_out,
                       rms_lm_head_intermediates=rms_lm_head_intermediates, logits=logits)
        for name, t in tensors.items():
            if t.device.type != "cuda" or not t.is_contiguous():
                raise RuntimeError(f"{name} must be a contiguous CUDA tensor")
            want = torch.int32 if name == "barriers" else torch.float32 if name.startswith("rope_") else torch.bfloat16
            if t.dtype != want:
                raise RuntimeError(f"{name} must be {want}")
        self._keep = tensors
        self.device = hidden_states.device
        L, qkv_rows, H = qkv_w.shape
        T, hkv, D = k_cache.shape[-3:]
        kv_batch = k_cache.shape[0] // L if k_cache.ndim == 4 else k_cache.shape[1]
        hq = qkv_rows // D - 2 * hkv
        if barriers.ndim != 4 or barriers.shape[0] != L or barriers.shape[1] != 10 or barriers.shape[2] != batch_size:
            raise RuntimeError("barriers must be int32 [layers, 10, batch_size, columns]")
        for name, width in (("hidden_states", H), ("rms_rope_intermediates", H), ("rms_gate_intermediates", H),
                            ("rms_lm_head_intermediates", H), ("post_ln_rope_q", hq * D), ("attn_out", hq * D),
                            ("silu_out", up_w.shape[1]), ("logits", lm_head_w.shape[0])):
            if tuple(tensors[name].shape) != (batch_size, width):
                raise RuntimeError(f"{name} must be [{batch_size}, {width}], got {tuple(tensors[name].shape)}")
        d = _lib.MkModelDesc()
        d.abi_version, d.weight_format = _lib.MK_ABI_VERSION, _lib.MK_WEIGHTS_BF16
        d.hidden_size, d.num_layers, d.num_q_heads, d.num_kv_heads, d.head_dim = H, L, hq, hkv, D
        d.intermediate_size, d.vocab_size = up_w.shape[1], lm_head_w.shape[0]
        d.attn_scale, d.rms_norm_eps = float(attn_scale), float(rms_norm_eps)
        d.qkv_w, d.o_w, d.up_w, d.gate_w = qkv_w.data_ptr(), o_w.data_ptr(), up_w.data_ptr(), gate_w.data_ptr()
        d.down_w, d.lm_head_w = down_w.data_ptr(), lm_head_w.data_ptr()
        d.attn_norm_w, d.mlp_norm_w, d.lm_head_norm_w = attn_norm_w.data_ptr(), mlp_norm_w.data_ptr(), lm_head_norm_w.data_ptr()
        d.embed_w = lm_head_w.data_ptr()  # required by the descriptor, never read: the set starts from hidden_states
        d.k_cache, d.v_cache, d.kv_batch, d.kv_max_len = k_cache.data_ptr(), v_cache.data_ptr(), kv_batch, T
        d.rope_cos, d.rope_sin, d.rope_positions = rope_cos.data_ptr(), rope_sin.data_ptr(), rope_cos.shape[0]
        d.hidden_states, d.logits = hidden_states.data_ptr(), logits.data_ptr()
        b = _lib.MkThroughputBuffers()
        b.rms_rope_intermediates, b.rms_gate_intermediates = rms_rope_intermediates.data_ptr(), rms_gate_intermediates.data_ptr()
        b.rms_lm_head_intermediates, b.post_ln_rope_q = rms_lm_head_intermediates.data_ptr(), post_ln_rope_q.data_ptr()
        b.attn_out, b.silu_out, b.barriers = attn_out.data_ptr(), silu_out.data_ptr(), barriers.data_ptr()
        b.barrier_cols, b.batch_size = barriers.shape[3], batch_size
        self.lib = _lib.load()
        self.handle = C.c_void_p()
        self._schedule_key = None
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_batched_create(C.byref(d), 128, C.byref(self.handle)))
            try:
                _lib.check(self.lib.mk_throughput_bind(self.handle, C.byref(b)))
            except Exception:
                self.close()
                raise

    def set_schedule(self, instructions: torch.Tensor) -> None:
        if instructions.device != self.device or instructions.dtype != torch.int32 or instructions.ndim != 3 \
                or instructions.shape[2] != 32 or not instructions.is_contiguous():
            raise RuntimeError("instructions must be a contiguous int32 [workers, queue_len, 32] tensor on the model's device")
        key = (instructions.data_ptr(), tuple(instructions.shape), instructions._version)
        if key == self._schedule_key:
            return
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_throughput_set_schedule(self.handle, instructions.data_ptr(), instructions.shape[0],
                                                           instructions.shape[1]))
        self._schedule_key = key

    def step(self, pos_id: int, stream=None) -> None:
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_step_throughput(self.handle, int(pos_id), st.cuda_stream))

    def status(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_batched_status(self.handle, torch.cuda.current_stream(self.device).cuda_stream))

    def close(self) -> None:
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.mk_batched_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Fp4Chain:
    """A prepared chain of NVFP4 x NVFP4 linears (``mk_fp4_chain_*``), the
    counterpart of the reference's ``vm_prepare`` / ``vm_run`` / ``vm_destroy``
    (``experimental/native_fp4_vm/vm.cu:14-63``).

    ``weights``: list of ``Nvfp4Native``; ``inputs`` / ``outputs``: bf16 CUDA
    tensors ``[batch, k_i]`` / ``[batch, m_i]`` (``outputs[i] is inputs[i + 1]``
    makes the chain dependent); ``input_scales``: tensor scale of each input's
    on-the-fly quantisation."""

    def __init__(self, weights, inputs, outputs, input_scales):
        import ctypes as C

        if not (len(weights) == len(inputs) == len(outputs) == len(input_scales)) or not weights:
            raise ValueError("weights, inputs, outputs and input_scales must be non-empty lists of one length")
        batch = inputs[0].shape[0]
        ops = (_lib.MkFp4ChainOperand * len(weights))()
        for i, (w, x, y, ts) in enumerate(zip(weights, inputs, outputs, input_scales)):
            for name, t, width in (("input", x, w.k), ("output", y, w.rows)):
                if t.device.type != "cuda" or t.dtype != torch.bfloat16 or not t.is_contiguous() or tuple(t.shape) != (batch, width):
                    raise ValueError(f"{name} {i} must be a contiguous bf16 CUDA tensor [{batch}, {width}]")
            ops[i].input, ops[i].output = x.data_ptr(), y.data_ptr()
            ops[i].w_packed, ops[i].w_scales_native = w.packed.data_ptr(), w.scales.data_ptr()
            ops[i].m, ops[i].k = w.rows, w.k
            ops[i].input_tensor_scale, ops[i].alpha = float(ts), float(w.tensor_scale) * float(ts)
        self._keep = (weights, inputs, outputs)
        self.device = inputs[0].device
        self.lib = _lib.load()
        self.handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_fp4_chain_prepare(ops, len(weights), batch, 1, C.byref(self.handle)))

    def run(self, stream=None) -> None:
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_fp4_chain_run(self.handle, st.cuda_stream))

    def status(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_fp4_chain_status(self.handle, torch.cuda.current_stream(self.device).cuda_stream))

    def close(self) -> None:
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.mk_fp4_chain_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
