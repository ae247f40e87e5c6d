"""Greedy decode loops (reference ``megakernels/generators.py:11-163``).

``output_tokens`` is a ``[1, n]`` tensor that already holds the first generated
token at column ``ntok_already_generated - 1``; ``generate`` fills the next
``ntok`` columns.  The token at column ``c`` is fed at position
``prompt_len + c`` of the cache.

* ``PyTorchGenerator`` - the model's plain PyTorch forward.
* ``MK_Generator``     - the reference's per-token protocol around the native
  step: host embedding lookup, counter reset, native call, ``torch.argmax``.
* ``MK_FusedGenerator`` - same results; embedding, counter reset and argmax
  happen inside the kernel and the whole chunk is enqueued without host
  synchronisation.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .mk import MK_Interpreter
from .model_types import BatchState
from .scheduler import Schedule


class Generator:
    def generate(self, output_tokens: Tensor, prompt_len: int, ntok: int, ntok_already_generated: int = 1):
        raise NotImplementedError

    def generate_with_eos(self, output_tokens: Tensor, prompt_len: int, ntok: int,
                          eos_token_check_interval: int, eos_token_ids: list[int]):
        """Generate in chunks, looking for an end-of-sequence token after each.
        Returns (column of the first EOS or ``ntok``, number of tokens generated)."""
        assert output_tokens.shape[0] == 1, "batch size must be 1"
        for done in range(1, ntok, eos_token_check_interval):
            chunk = min(eos_token_check_interval, ntok - done)
            self.generate(output_tokens, prompt_len=prompt_len, ntok=chunk, ntok_already_generated=done)
            host = output_tokens[0, done : done + chunk].cpu()
            for j, tok in enumerate(host):
                if tok in eos_token_ids:
                    return done + j, done + chunk - 1
        return ntok, ntok - 1


class PyTorchGenerator(Generator):
    def __init__(self, model):
        self.model = model

    def generate(self, output_tokens: Tensor, prompt_len: int, ntok: int, ntok_already_generated: int = 1):
        bs = output_tokens.shape[0]
        seq0 = prompt_len + ntok_already_generated
        for i in range(ntok):
            col = ntok_already_generated + i - 1
            pos = torch.full((bs, 1), seq0 - 1 + i, dtype=torch.long, device=self.model.device)
            out = self.model(BatchState(input_ids=output_tokens[:, col : col + 1], position_ids=pos, seq_len=seq0 + i))
            output_tokens[:, col + 1] = out.output_ids.squeeze(-1)


class MK_Generator(Generator):
    def __init__(self, model, interpreter: MK_Interpreter, schedule: Schedule, barrier_fill_val: int = 0,
                 skip_mk: bool = False, skip_rest: bool = False):
        self.model = model
        self.interpreter = interpreter
        self.schedule = schedule
        self.barrier_fill_val = barrier_fill_val
        self.skip_mk = skip_mk
        self.skip_rest = skip_rest
        self.fill()

    def fill(self):
        self.schedule.globs.barriers.fill_(self.barrier_fill_val)

    def replace_with_noops(self):
        self.schedule.globs.instructions.zero_()

    def run(self, input_ids: Tensor, pos_id: int):
        globs = self.schedule.globs
        if not self.skip_rest:
            embedded = self.model.model.embed_tokens(BatchState(input_ids=input_ids))
            globs.hidden_states[:] = embedded.hidden_states.squeeze(1)
        self.fill()
        globs.pos_id = pos_id
        if not self.skip_mk:
            self.interpreter.interpret(globs)
        if self.skip_rest:
            return input_ids
        return torch.argmax(globs.logits, dim=-1)

    def generate(self, output_tokens: Tensor, prompt_len: int, ntok: int, ntok_already_generated: int = 1):
        for i in range(ntok):
            col = ntok_already_generated + i - 1
            out = self.run(output_tokens[:, col : col + 1], pos_id=prompt_len + col)
            output_tokens[:, col + 1] = out.squeeze(-1)


class MK_FusedGenerator(Generator):
    """Decode loop with no per-token host work beyond one launch."""

    def __init__(self, model, schedule: Schedule, quantized: dict | None = None):
        """``quantized``: result of ``nvfp4.quantize_model(model)`` to decode with
        NVFP4 weight-only linears instead of the bf16 weights."""
        from .runtime import Megakernel

        self.model = model
        self.schedule = schedule
        globs = schedule.globs
        if globs.instructions is None:
            raise ValueError("schedule has no instruction tensor; call tensorize_instructions first")
        self.mk = Megakernel.from_globals(globs, embed_w=model.model.embed_tokens.embed_tokens.weight.data,
                                          quantized=quantized)
        globs.barriers.zero_()
        self._prefiller = None

    def prefill(self, prompt: Tensor, start_pos: int = 0) -> Tensor:
        """Process the prompt (1-D token ids on the model's device) on the GPU's
        batched tensor-core path instead of the PyTorch forward the reference uses
        (megakernels/scripts/generate.py:125-132): fills cache slot 0 at positions
        ``start_pos ..`` and returns the first generated token (1-element int32
        tensor).  Runs with the bf16 weights also when decoding is NVFP4."""
        if self._prefiller is None:
            from .batched import BatchedDecoder

            self._prefiller = BatchedDecoder(self.model, max_batch=128)
        return self._prefiller.prefill(prompt.to(torch.int32).contiguous(), slot=0, start_pos=start_pos)

    def generate(self, output_tokens: Tensor, prompt_len: int, ntok: int, ntok_already_generated: int = 1):
        assert output_tokens.shape[0] == 1, "batch size must be 1"
        col = ntok_already_generated - 1
        first = output_tokens[0, col : col + 1].to(torch.int32)
        produced = torch.empty(ntok, dtype=torch.int32, device=output_tokens.device)
        self.mk.decode(first, produced, start_pos=prompt_len + col, count=ntok)
        output_tokens[0, col + 1 : col + 1 + ntok] = produced.to(output_tokens.dtype)
        self.schedule.globs.pos_id = prompt_len + col + ntok - 1
