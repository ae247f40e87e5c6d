"""Python handle over the C-ABI decode megakernel.

``Megakernel`` binds one ``Globals`` (weights, cache, activation buffers,
instruction queues) to a library handle once and then launches decode steps by
position id.  It is what the ``mk_llama`` shim and ``MK_Generator`` call; see
``include/b200_megakernel.h`` for the functions underneath.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import (
    MK_STEP_EMBED,
    MK_STEP_RESET_BARRIERS,
    MK_STEP_TIMINGS,
    MK_STEP_WRITE_TOKEN,
    MegakernelError,
)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require(t: torch.Tensor, name: str, dtype: torch.dtype):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a tensor")
    if t.device.type != "cuda":
        raise RuntimeError(f"{name} must live on a CUDA device (the decode step has no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


class Megakernel:
    """One bound model.  Tensors are borrowed: keep them alive while this lives."""

    def __init__(
        self,
        *,
        barriers, qkv_w, attn_norm_w, o_w, mlp_norm_w, up_w, gate_w, down_w, lm_head_norm_w, lm_head_w,
        k_cache, v_cache, rope_cos, rope_sin, hidden_states, q_post_rope, attn_out,
        attn_lse_intermediates, attn_out_intermediates, silu_out, logits,
        attn_scale: float, rms_norm_eps: float, skip_attn_reduction: bool = True,
        embed_w=None, num_kv_heads: int | None = None, quantized: dict | None = None,
    ):
        """``quantized``: for an NVFP4 weight-only model, a dict with lists of
        ``Nvfp4Weight`` per layer under ``qkv``, ``o``, ``up``, ``gate``, ``down`` and
        one under ``lm_head``; the bf16 weight arguments then only supply shapes
        and may be dropped by the caller afterwards."""
        bf16, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        weights = dict(qkv_w=qkv_w, o_w=o_w, up_w=up_w, gate_w=gate_w, down_w=down_w, lm_head_w=lm_head_w)
        if quantized is None:
            for name, t in weights.items():
                _require(t, name, bf16)
        for name, t in dict(attn_norm_w=attn_norm_w, mlp_norm_w=mlp_norm_w, lm_head_norm_w=lm_head_norm_w,
                            k_cache=k_cache, v_cache=v_cache, hidden_states=hidden_states,
                            q_post_rope=q_post_rope, attn_out=attn_out, silu_out=silu_out, logits=logits).items():
            _require(t, name, bf16)
        for name, t in dict(rope_cos=rope_cos, rope_sin=rope_sin, attn_lse_intermediates=attn_lse_intermediates,
                            attn_out_intermediates=attn_out_intermediates).items():
            _require(t, name, f32)
        _require(barriers, "barriers", i32)
        if embed_w is not None:
            _require(embed_w, "embed_w", bf16)
        if qkv_w.ndim != 3 or down_w.ndim != 3 or barriers.ndim != 3:
            raise ValueError("stacked weights and barriers must be 3-D")
        if k_cache.ndim not in (4, 5) or k_cache.shape != v_cache.shape:
            raise ValueError("k_cache/v_cache must be [L,B,T,Hkv,D] or [(L B),T,Hkv,D] and equal in shape")

        layers, qkv_rows, hidden = qkv_w.shape
        inter = down_w.shape[2]
        head_dim = k_cache.shape[-1]
        kv_heads = k_cache.shape[-2]
        kv_len = k_cache.shape[-3]
        kv_batch = k_cache.shape[1] if k_cache.ndim == 5 else k_cache.shape[0] // layers
        q_heads = qkv_rows // head_dim - 2 * kv_heads
        if num_kv_heads is not None and num_kv_heads != kv_heads:
            raise ValueError("num_kv_heads disagrees with the cache shape")

        self._keep = [barriers, qkv_w, attn_norm_w, o_w, mlp_norm_w, up_w, gate_w, down_w, lm_head_norm_w, lm_head_w,
                      k_cache, v_cache, rope_cos, rope_sin, hidden_states, q_post_rope, attn_out,
                      attn_lse_intermediates, attn_out_intermediates, silu_out, logits, embed_w]
        self.device = qkv_w.device
        self.lib = _lib.load()
        d = _lib.MkModelDesc()
        d.abi_version = _lib.MK_ABI_VERSION
        d.weight_format = _lib.MK_WEIGHTS_BF16 if quantized is None else _lib.MK_WEIGHTS_NVFP4
        d.hidden_size, d.num_layers, d.num_q_heads, d.num_kv_heads = hidden, layers, q_heads, kv_heads
        d.head_dim, d.intermediate_size, d.vocab_size = head_dim, inter, lm_head_w.shape[0]
        d.attn_scale, d.rms_norm_eps = float(attn_scale), float(rms_norm_eps)
        if quantized is None:
            d.qkv_w, d.o_w, d.up_w, d.gate_w, d.down_w = map(_ptr, (qkv_w, o_w, up_w, gate_w, down_w))
            d.lm_head_w = _ptr(lm_head_w)
        else:
            self._tables = {}
            for key, field in (("qkv", "qkv_q"), ("o", "o_q"), ("up", "up_q"), ("gate", "gate_q"), ("down", "down_q"),
                               ("lm_head", "lm_head_q")):
                mats = quantized[key] if key != "lm_head" else [quantized[key]]
                if key != "lm_head" and len(mats) != layers:
                    raise ValueError(f"quantized[{key!r}] needs one matrix per layer")
                table = (_lib.MkNvfp4Matrix * len(mats))()
                for i, m in enumerate(mats):
                    table[i].packed, table[i].scales = m.packed.data_ptr(), m.scales.data_ptr()
                    table[i].tensor_scale = float(m.tensor_scale)
                self._tables[key] = (table, mats)  # keep the ctypes arrays and the tensors alive
                setattr(d, field, table)
        d.attn_norm_w, d.mlp_norm_w = map(_ptr, (attn_norm_w, mlp_norm_w))
        d.lm_head_norm_w, d.embed_w = _ptr(lm_head_norm_w), _ptr(embed_w)
        d.k_cache, d.v_cache, d.kv_batch, d.kv_max_len = _ptr(k_cache), _ptr(v_cache), kv_batch, kv_len
        d.rope_cos, d.rope_sin, d.rope_positions = _ptr(rope_cos), _ptr(rope_sin), rope_cos.shape[0]
        d.hidden_states, d.q_post_rope, d.attn_out = map(_ptr, (hidden_states, q_post_rope, attn_out))
        d.attn_lse_intermediates = _ptr(attn_lse_intermediates)
        d.attn_out_intermediates = _ptr(attn_out_intermediates)
        d.max_partials = attn_lse_intermediates.shape[1]
        d.silu_out, d.logits = _ptr(silu_out), _ptr(logits)
        d.barriers, d.barrier_rows, d.barrier_cols = _ptr(barriers), barriers.shape[1], barriers.shape[2]
        d.skip_attn_reduction = int(bool(skip_attn_reduction))
        self.desc = d
        self.handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_create(C.byref(d), C.byref(self.handle)))
        self._schedule_key = None
        self.token_cell = torch.zeros(2, dtype=torch.int32, device=self.device)

    # -- construction from the schedule's table ---------------------------
    @classmethod
    def from_globals(cls, globs, embed_w=None, quantized: dict | None = None) -> "Megakernel":
        mk = cls(
            barriers=globs.barriers, qkv_w=globs.qkv_proj_weights, attn_norm_w=globs.attn_ln_weights,
            o_w=globs.o_proj_weights, mlp_norm_w=globs.mlp_ln_weights, up_w=globs.up_proj_weights,
            gate_w=globs.gate_proj_weights, down_w=globs.down_proj_weights,
            lm_head_norm_w=globs.lm_head_norm_weights.data, lm_head_w=globs.lm_head_weights.data,
            k_cache=globs.k_cache, v_cache=globs.v_cache, rope_cos=globs.rope_cos, rope_sin=globs.rope_sin,
            hidden_states=globs.hidden_states, q_post_rope=globs.post_ln_rope_q, attn_out=globs.attn_out,
            attn_lse_intermediates=globs.attn_lse_intermediates,
            attn_out_intermediates=globs.attn_out_intermediates, silu_out=globs.silu_out, logits=globs.logits,
            attn_scale=globs.attn_scale, rms_norm_eps=globs.rms_norm_eps,
            skip_attn_reduction=globs.skip_attn_reduction, embed_w=embed_w, quantized=quantized,
        )
        if globs.instructions is not None:
            mk.set_schedule(globs.instructions, globs.timings)
        return mk

    def set_schedule(self, instructions: torch.Tensor, timings: torch.Tensor | None):
        _require(instructions, "instructions", torch.int32)
        if instructions.ndim != 3 or instructions.shape[2] != 32:
            raise ValueError("instructions must be int32 [workers, queue_len, 32]")
        if timings is not None:
            _require(timings, "timings", torch.int32)
            if tuple(timings.shape) != (instructions.shape[0], instructions.shape[1], 128):
                raise RuntimeError("instruction/timing queue dimensions do not match worker grid")
        # the library inspects the queues when they are set: an in-place rewrite counts as a new schedule
        key = (instructions.data_ptr(), _ptr(timings), tuple(instructions.shape), instructions._version)
        if key == self._schedule_key:
            return
        _lib.check(self.lib.mk_set_schedule(self.handle, instructions.data_ptr(), _ptr(timings),
                                            instructions.shape[0], instructions.shape[1]))
        self._schedule_key = key
        self._keep_schedule = (instructions, timings)

    # -- stepping -----------------------------------------------------------
    def step(self, pos_id: int, *, flags: int = 0, token_in: torch.Tensor | None = None,
             token_out: torch.Tensor | None = None, stream: torch.cuda.Stream | None = None):
        stream = stream or torch.cuda.current_stream(self.device)
        _lib.check(self.lib.mk_step(self.handle, int(pos_id), int(flags), _ptr(token_in), _ptr(token_out),
                                    stream.cuda_stream))

    def decode(self, first_token: torch.Tensor, tokens_out: torch.Tensor, start_pos: int, count: int,
               stream: torch.cuda.Stream | None = None):
        """``count`` greedy steps with no host round trip between them: step i reads
        its input token from where step i-1 wrote its argmax, embeds it in-kernel and
        resets the dependency counters itself.  ``tokens_out`` is an int32 device
        vector of at least ``count`` cells; ``first_token`` a 1-element int32 tensor."""
        if self.desc.embed_w is None:
            raise RuntimeError("decode() needs the embedding table (embed_w)")
        flags = MK_STEP_EMBED | MK_STEP_RESET_BARRIERS | MK_STEP_WRITE_TOKEN
        stream = stream or torch.cuda.current_stream(self.device)
        base = tokens_out.data_ptr()
        src = first_token.data_ptr()
        for i in range(count):
            dst = base + 4 * i
            _lib.check(self.lib.mk_step(self.handle, start_pos + i, flags, src, dst, stream.cuda_stream))
            src = dst

    def query(self) -> dict:
        info = _lib.MkLaunchInfo()
        _lib.check(self.lib.mk_query(self.handle, C.byref(info)))
        out = {name: getattr(info, name) for name, _ in info._fields_}
        out["cooperative_launch"] = bool(out["cooperative_launch"])
        out["page_count"], out["page_size"] = out["stage_count"], out["stage_bytes"]
        return out

    def status(self, stream: torch.cuda.Stream | None = None) -> dict:
        """Synchronise and return the device status words; raises
        ``MegakernelError`` (code MK_ERR_DEVICE_WAIT) if a bounded wait expired."""
        stream = stream or torch.cuda.current_stream(self.device)
        st = _lib.MkStatus()
        code = self.lib.mk_status(self.handle, C.byref(st), stream.cuda_stream)
        out = {name: getattr(st, name) for name, _ in st._fields_}
        if code != 0:
            err = MegakernelError(code, self.lib.mk_last_error().decode())
            err.status = out
            raise err
        return out

    def stuck_warps(self, max_records: int = 2048) -> list[dict]:
        """After ``status()`` raised: the bounded wait every waiting warp was in
        (worker, warp, code, opcode, slot, detail)."""
        buf = (C.c_int32 * (6 * max_records))()
        n = C.c_int32(0)
        _lib.check(self.lib.mk_status_detail(self.handle, buf, max_records, C.byref(n)))
        names = ("worker", "warp", "code", "opcode", "slot", "detail")
        return [dict(zip(names, buf[6 * i : 6 * i + 6])) for i in range(min(n.value, max_records))]

    # -- tensor parallelism ------------------------------------------------
    def tp_init(self, rank: int, world: int, vocab_offset: int) -> bytes:
        """Allocates this GPU's exchange buffer; returns its CUDA IPC handle (64
        bytes) for the caller to all-gather across the ranks."""
        buf = C.create_string_buffer(_lib.MK_TP_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.mk_tp_init(self.handle, int(rank), int(world), int(vocab_offset), buf))
        return bytes(buf.raw)

    def tp_connect(self, handles: list[bytes]):
        """Maps the peers' exchange buffers; ``handles`` in rank order."""
        if any(len(h) != _lib.MK_TP_HANDLE_BYTES for h in handles):
            raise ValueError("every IPC handle must be 64 bytes")
        blob = C.create_string_buffer(b"".join(handles), len(handles) * _lib.MK_TP_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            # the library checks the count against the world size given to tp_init
            _lib.check(self.lib.mk_tp_connect(self.handle, blob, len(handles)))

    def set_wait_budget(self, cycles: int):
        _lib.check(self.lib.mk_set_wait_budget(self.handle, int(cycles)))

    def set_option(self, option: int, value: int):
        _lib.check(self.lib.mk_set_option(self.handle, int(option), int(value)))

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.mk_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


__all__ = ["Megakernel", "MegakernelError", "MK_STEP_EMBED", "MK_STEP_RESET_BARRIERS", "MK_STEP_WRITE_TOKEN",
           "MK_STEP_TIMINGS"]
