"""Schedule builder for batch-1 decode: buffers, per-op work splits and the
layer DAG.

Follows ``megakernels/demos/latency/scheduler.py`` of the reference:
``pick_num_attention_partitions`` (:21-35), ``make_globals`` (:38-115), the
work splits ``schedule_qkv`` / ``schedule_upgate`` / ``schedule_downproj`` /
``schedule_lm_head`` (:118-232) and ``make_dag`` / ``make_dag_layer``
(:235-395).  With ``skip_attn_reduction=True`` (the reference's only mode) the
DAG is node-for-node the reference's.  With ``skip_attn_reduction=False`` the
cache is split into ``globs.num_attention_partitions`` slices per KV head and
one terminal ``AttentionReduction`` per KV head merges them; the reference
defines both instructions but never schedules the pair.
"""
from __future__ import annotations

import math

import torch

from ...instructions import NoOp
from ...scheduler import DAG_Node, INTS_PER_INSTRUCTION, ScheduleBuilder
from ...utils import assert_div, get_sm_count
from .instructions import (
    AttentionReduction,
    DownProjResidual,
    Globals,
    LayerNorm_QKV_MatVecRopeAppend,
    LayerNormDoubleMatVecSiLU,
    O_ProjResidual,
    PartialAttention,
    RMS_LM_Head,
)

# A terminal reduction lists every partial in one 32-word instruction:
# opcode + 5 scalar words + list + output slot.
MAX_ATTENTION_PARTITIONS = 24


def pick_num_attention_partitions(prompt_len: int, ntok: int, device=None) -> int:
    """At least 256 cached tokens per slice, at most 24 slices."""
    slices = math.ceil((prompt_len + ntok) / 256)
    return max(1, min(slices, MAX_ATTENTION_PARTITIONS))


def make_globals(model, skip_attn_reduction: bool = True, num_attention_partitions: int = 1) -> Globals:
    cfg = model.config
    device, dtype = model.device, model.dtype

    def zeros(shape, dt=dtype):
        return torch.zeros(shape, device=device, dtype=dt)

    sp = model.stacked_params
    max_partials = get_sm_count(device)
    total_heads = cfg.num_attention_heads + 2 * cfg.num_key_value_heads

    globs = Globals(
        qkv_proj_weights=sp.qkv_proj,
        attn_ln_weights=sp.attn_ln_weight,
        o_proj_weights=sp.o_proj,
        mlp_ln_weights=sp.mlp_ln_weight,
        up_proj_weights=sp.up_proj,
        gate_proj_weights=sp.gate_proj,
        down_proj_weights=sp.down_proj,
        lm_head_norm_weights=model.lm_head.input_norm.weight,
        lm_head_weights=model.lm_head.lm_head.weight,
        k_cache=model.stacked_kv_cache[0],
        v_cache=model.stacked_kv_cache[1],
        rope_cos=model.model.rope_cos,
        rope_sin=model.model.rope_sin,
        num_hidden_layers=cfg.num_hidden_layers,
        num_attention_heads=cfg.num_attention_heads,
        num_kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim,
        hidden_size=cfg.hidden_size,
        intermediate_size=cfg.intermediate_size,
        vocab_size=cfg.vocab_size,
        attn_scale=1 / math.sqrt(cfg.head_dim),
        rms_norm_eps=cfg.rms_norm_eps,
        device=device,
        hidden_states=zeros(cfg.hidden_size),
        # one counter row per opcode (10 > number of opcodes), one column per Q/K/V head
        barriers=zeros([cfg.num_hidden_layers, 10, total_heads], torch.int32),
        pos_id=0,
        post_ln_rope_q=zeros(cfg.num_attention_heads * cfg.head_dim),
        attn_out=zeros(cfg.num_attention_heads * cfg.head_dim),
        attn_lse_intermediates=zeros([cfg.num_attention_heads, max_partials], torch.float32),
        attn_out_intermediates=zeros([cfg.num_attention_heads, max_partials, cfg.head_dim], torch.float32),
        silu_out=zeros(cfg.intermediate_size),
        logits=zeros(cfg.vocab_size),
        skip_attn_reduction=skip_attn_reduction,
        up_gate_proj_block_size=16,
        down_proj_block_size=16,
        o_proj_block_size=16,
        lm_head_block_size=16,
        matvec_reduction_size=down_slice_width(cfg.intermediate_size),
        qkv_block_size=16,
        attn_kv_block_size=16,
        attn_reduction_size=4,
    )
    globs.num_attention_partitions = 1 if skip_attn_reduction else num_attention_partitions
    return globs


def down_slice_width(intermediate_size: int) -> int:
    """Columns of one down-projection slice: 2048 (the reference's
    ``matvec_reduction_size``) when it divides ``intermediate_size``, else the
    widest multiple of 256 below it that does (a tensor-parallel share of the
    FFN, e.g. 1792 for 14336/2).  The kernel applies the same rule."""
    for width in range(2048, 0, -256):
        if intermediate_size % width == 0:
            return width
    raise ValueError(f"intermediate_size {intermediate_size} is not a multiple of 256")


def _even_ranges(num_blocks: int, workers: int):
    """Contiguous block ranges whose sizes differ by at most one.  With fewer
    blocks than workers (small tensor-parallel shares) every block is its own range."""
    per = num_blocks / workers
    if per <= 1:
        return [(b, b + 1) for b in range(num_blocks)]
    return [(round(w * per), round((w + 1) * per)) for w in range(workers)]


def schedule_qkv(globs: Globals, layer_idx: int):
    rows = (globs.num_attention_heads + 2 * globs.num_kv_heads) * globs.head_dim
    blocks = assert_div(rows, globs.qkv_block_size)
    return [
        LayerNorm_QKV_MatVecRopeAppend(layer_idx, start, end)
        for start, end in _even_ranges(blocks, globs.sm_count())
    ]


def schedule_upgate(globs: Globals, layer_idx: int):
    blocks = assert_div(globs.intermediate_size, globs.up_gate_proj_block_size)
    workers = globs.sm_count()
    room = INTS_PER_INSTRUCTION - 3  # opcode, layer and list length take three words
    out = []
    for w in range(min(workers, blocks)):
        mine = list(range(w, blocks, workers))
        for i in range(0, len(mine), room):
            out.append(LayerNormDoubleMatVecSiLU(layer_idx, mine[i : i + room]))
    return out


def schedule_downproj(globs: Globals, layer_idx: int):
    """(column slice, row block) jobs in column-major order, dealt out evenly;
    an instruction never straddles two column slices."""
    row_blocks = assert_div(globs.hidden_size, globs.down_proj_block_size)
    # 2048-column slices of the input; equals intermediate_size // hidden_size (the
    # reference's expression) whenever hidden_size is 2048
    col_slices = assert_div(globs.intermediate_size, globs.matvec_reduction_size)
    workers = globs.sm_count()
    jobs = [(c, r) for c in range(col_slices) for r in range(row_blocks)]

    out = []
    taken = 0
    for w in range(workers):
        if taken == len(jobs):
            break
        share = max(1.0, (len(jobs) - taken) / (workers - w))
        chunk = jobs[taken : taken + round(share)]
        col = chunk[0][0]
        chunk = [j for j in chunk if j[0] == col]
        first = chunk[0][1]
        assert [j[1] for j in chunk] == list(range(first, first + len(chunk)))
        out.append(DownProjResidual(layer_idx, first, first + len(chunk), col))
        taken += len(chunk)
    return out


def schedule_downproj_rows_together(globs: Globals, layer_idx: int):
    """Every worker gets a contiguous range of output row blocks and ALL column
    slices of it, listed slice 0, 1, ... one after the other.  Same instruction
    type and wire format as ``schedule_downproj``; with the ``rrk`` assignment a
    worker then adds its slices to the residual stream by itself, in the
    interpreter's slice order, instead of handing partial sums to another SM.
    Not a reference layout (its down projection always splits rows AND columns
    across workers, ``latency/scheduler.py:165-199``)."""
    row_blocks = assert_div(globs.hidden_size, globs.down_proj_block_size)
    col_slices = assert_div(globs.intermediate_size, globs.matvec_reduction_size)
    out = []
    for start, end in _even_ranges(row_blocks, globs.sm_count()):
        if end > start:
            out.extend(DownProjResidual(layer_idx, start, end, c) for c in range(col_slices))
    return out


def schedule_lm_head(globs: Globals):
    blocks = assert_div(globs.vocab_size, globs.lm_head_block_size)
    return [RMS_LM_Head(start, end) for start, end in _even_ranges(blocks, globs.sm_count())]


def make_dag(globs: Globals, stop_after_op: str | None = None, layer_limit: int | None = None, first_layer: int = 0):
    """``layer_limit`` and ``stop_after_op`` cut the schedule short as in the
    reference; ``first_layer`` (not in the reference) starts it at a later layer,
    whose input is then ``hidden_states`` as given: one layer can be run alone
    from a recorded residual stream."""
    layers = globs.num_hidden_layers if layer_limit is None else layer_limit
    nodes: list[DAG_Node] = []
    frontier: list[DAG_Node] = []
    for layer in range(first_layer, layers):
        added, frontier = make_dag_layer(globs, layer, frontier, stop_after_op)
        nodes.extend(added)

    if layers == globs.num_hidden_layers:
        head = [DAG_Node(ins, frontier) for ins in schedule_lm_head(globs)]
        nodes.extend(head)
        frontier = head

    return nodes, DAG_Node(NoOp(), frontier)


def make_dag_layer(globs: Globals, layer_idx: int, prev_layer_outputs: list[DAG_Node], stop_after_op: str | None = None):
    partitions = 1 if globs.skip_attn_reduction else int(getattr(globs, "num_attention_partitions", 1))
    if not 1 <= partitions <= MAX_ATTENTION_PARTITIONS:
        raise ValueError(f"num_attention_partitions must be in 1..{MAX_ATTENTION_PARTITIONS}")
    nodes: list[DAG_Node] = []

    # -- fused QKV -------------------------------------------------------
    qkv_nodes = [DAG_Node(ins, prev_layer_outputs) for ins in schedule_qkv(globs, layer_idx)]
    producer_of_block = {}
    for n in qkv_nodes:
        for b in n.instruction.block_indices():
            producer_of_block[b] = n
    nodes.extend(qkv_nodes)
    if stop_after_op == "qkv":
        return nodes, qkv_nodes

    # -- attention -------------------------------------------------------
    blocks_per_head = assert_div(globs.head_dim, globs.qkv_block_size)
    group = globs.num_attention_heads // globs.num_kv_heads
    attn_nodes: list[DAG_Node] = []
    for kv_head in range(globs.num_kv_heads):
        k_head = globs.num_attention_heads + kv_head
        v_head = k_head + globs.num_kv_heads
        needed = list(range(kv_head * group * blocks_per_head, (kv_head + 1) * group * blocks_per_head))
        needed += list(range(k_head * blocks_per_head, (k_head + 1) * blocks_per_head))
        needed += list(range(v_head * blocks_per_head, (v_head + 1) * blocks_per_head))
        deps = list({producer_of_block[b] for b in needed})
        for part in range(partitions):
            attn_nodes.append(DAG_Node(PartialAttention(layer_idx, kv_head, partitions, part), deps))
    nodes.extend(attn_nodes)
    if stop_after_op == "partial":
        return nodes, attn_nodes

    attn_done = attn_nodes
    if not globs.skip_attn_reduction:
        if group != globs.attn_reduction_size:
            raise ValueError("attention reduction merges exactly one KV head's query group")
        merge_nodes = []
        for kv_head in range(globs.num_kv_heads):
            parents = [n for n in attn_nodes if n.instruction.kv_head_idx == kv_head]
            ins = AttentionReduction(
                layer_idx=layer_idx,
                head_start_idx=kv_head * group,
                num_partials=partitions,
                is_terminal=True,
                reduction_list=list(range(partitions)),
                output_partial_idx=None,
            )
            merge_nodes.append(DAG_Node(ins, parents))
        nodes.extend(merge_nodes)
        attn_done = merge_nodes
        if stop_after_op == "reduction":
            return nodes, merge_nodes

    # -- output projection -------------------------------------------------
    o_blocks = assert_div(globs.hidden_size, globs.o_proj_block_size)
    o_nodes = [DAG_Node(O_ProjResidual(layer_idx, b, b + 1, 0), attn_done) for b in range(o_blocks)]
    nodes.extend(o_nodes)
    if stop_after_op == "oproj":
        return nodes, o_nodes

    # -- gate / up ---------------------------------------------------------
    upgate_nodes = [DAG_Node(ins, o_nodes) for ins in schedule_upgate(globs, layer_idx)]
    nodes.extend(upgate_nodes)
    if stop_after_op == "upgate":
        return nodes, upgate_nodes

    # -- down projection ---------------------------------------------------
    ordered = getattr(globs, "ordered_downproj", False)
    down_nodes: list[DAG_Node] = []
    together = getattr(globs, "down_rows_together", False)
    for ins in (schedule_downproj_rows_together if together else schedule_downproj)(globs, layer_idx):
        # An ordered bf16 reduction waits for the previous column slice.
        earlier = [n for n in down_nodes if ordered and n.instruction.reduction_block_idx == ins.reduction_block_idx - 1]
        down_nodes.append(DAG_Node(ins, upgate_nodes + earlier))
    nodes.extend(down_nodes)
    if stop_after_op not in (None, "downproj"):
        raise AssertionError(f"unknown stop_after_op {stop_after_op!r}")
    return nodes, down_nodes


class LatencyScheduleBuilder(ScheduleBuilder):
    @classmethod
    def make_globals(cls, model, skip_attn_reduction: bool = True, num_attention_partitions: int = 1):
        return make_globals(model, skip_attn_reduction, num_attention_partitions)

    @classmethod
    def make_dag(cls, globs, stop_after_op: str | None = None, layer_limit: int | None = None, first_layer: int = 0):
        return make_dag(globs, stop_after_op, layer_limit, first_layer)

    @classmethod
    def build(cls, model, stop_after_op=None, layer_limit=None, skip_attn_reduction: bool = True,
              num_attention_partitions: int = 1, first_layer: int = 0, down_rows_together: bool = False):
        """``down_rows_together``: lay the down projection out so that one worker
        owns all column slices of its output rows (``schedule_downproj_rows_together``;
        assign with policy ``rrk``).  The default is the reference's layout."""
        from ...scheduler import Schedule

        globs = cls.make_globals(model, skip_attn_reduction, num_attention_partitions)
        globs.down_rows_together = down_rows_together
        nodes, end = cls.make_dag(globs, stop_after_op, layer_limit, first_layer)
        return Schedule(globs, nodes, end)


def build_b200_schedule(model, **kwargs):
    """The schedule this library runs fastest: the reference's instruction set
    and per-op work splits, with the down projection laid out so that one SM owns
    all column slices of its output rows (``down_rows_together``) and the
    row-keeping round-robin assignment (``rrk``).  Returns a ``Schedule`` whose
    ``globs.instructions`` / ``globs.timings`` are already filled.  Keyword
    arguments go to ``LatencyScheduleBuilder.build``."""
    from ...scheduler import assign_to_sms, tensorize_instructions

    sched = LatencyScheduleBuilder.build(model, down_rows_together=True, **kwargs)
    tensorize_instructions(sched.globs, assign_to_sms("rrk", schedule=sched))
    return sched
