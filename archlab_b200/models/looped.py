"""Tied prelude / core / coda execution: a stack of blocks whose middle segment is run several times.

Semantics (src/archlab/architectures/prelude_loop_coda.py:16-49, src/archlab/automodel/deepseek_v41_loop.py,
behaviour pinned by the reference's tests/test_prelude_loop_coda.py): the prelude output is the *anchor*; the raw
prelude feeds the first core pass; after EVERY core pass (also the last, before the coda) the hidden state goes
through the parameter-free boundary ``rms_norm(h) + anchor / sqrt(2)`` (fp32 RMS over features, per stream).  Core
blocks are stored once and appear once in ``state_dict``; gradients of the repetitions accumulate into them.

Here the loop is an explicit module (``LoopedStack``) that owns the block list and runs it, instead of an execution
iterator patched over a module registry: each forward builds its own anchor as a local, so two live forward graphs
or an activation-checkpoint replay cannot see each other's anchor.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass(frozen=True)
class LoopLayout:
    prelude: int = 6
    core: int = 7
    coda: int = 7

    def __post_init__(self):
        for name in ("prelude", "core", "coda"):
            n = getattr(self, name)
            if type(n) is not int or n < 1:
                raise ValueError(f"{name} must be a positive integer block count")

    @property
    def stored_depth(self) -> int:
        return self.prelude + self.core + self.coda

    @property
    def segments(self) -> tuple[range, range, range]:
        a, b = self.prelude, self.prelude + self.core
        return range(0, a), range(a, b), range(b, self.stored_depth)

    def execution(self, repetitions: int) -> list[int]:
        """Stored-block index of every executed block, in order."""
        if type(repetitions) is not int or repetitions < 1:
            raise ValueError("recursion count must be a positive integer")
        pre, core, coda = self.segments
        return [*pre, *(list(core) * repetitions), *coda]

    def executed_depth(self, repetitions: int) -> int:
        return self.prelude + self.core * repetitions + self.coda


def balanced_layout(depth: int) -> LoopLayout:
    """Thirds of ``depth``; a remainder of one goes to the core, of two to core and coda."""
    third, rest = divmod(depth, 3)
    return LoopLayout(third, third + (rest >= 1), third + (rest == 2))


def boundary(hidden: torch.Tensor, anchor: torch.Tensor) -> torch.Tensor:
    normed = F.rms_norm(hidden.float(), (hidden.shape[-1],))
    return (normed + anchor.float() * (1.0 / math.sqrt(2.0))).to(hidden.dtype)


class LoopedStack(nn.Module):
    """``blocks`` stored once, executed as prelude, ``repetitions`` x core (boundary after each pass), coda.

    ``step(block, hidden, carry) -> (hidden, carry)`` adapts the block signature; ``carry`` is whatever else travels
    between blocks (KV / index ownership, mixing state).  Every core pass restarts from the carry the prelude
    handed over, because ownership follows the stored block, while the hidden state recurs."""

    def __init__(self, blocks: Sequence[nn.Module], layout: LoopLayout, *, repetitions: int = 2,
                 step: Callable | None = None):
        super().__init__()
        if len(blocks) != layout.stored_depth:
            raise ValueError(f"layout stores {layout.stored_depth} blocks, {len(blocks)} were given")
        self.blocks = blocks if isinstance(blocks, nn.ModuleList) else nn.ModuleList(blocks)
        self.layout = layout
        self.step = step or (lambda block, hidden, carry: (block(hidden), carry))
        self.set_repetitions(repetitions)
        self.visits = [0] * layout.stored_depth          # executions of each stored block in the last forward

    def set_repetitions(self, repetitions: int) -> None:
        self.layout.execution(repetitions)               # validates
        self.repetitions = repetitions

    def forward(self, hidden: torch.Tensor, carry=None):
        pre, core, coda = self.layout.segments
        visits = [0] * self.layout.stored_depth

        def run(indices, hidden, carry):
            for i in indices:
                hidden, carry = self.step(self.blocks[i], hidden, carry)
                visits[i] += 1
            return hidden, carry

        hidden, carry = run(pre, hidden, carry)
        anchor, carry_at_prelude = hidden, carry
        for _ in range(self.repetitions):
            hidden, carry = run(core, hidden, carry_at_prelude)
            hidden = boundary(hidden, anchor)
        hidden, carry = run(coda, hidden, carry)
        self.visits = visits
        return hidden if carry is None else (hidden, carry)


def loop_blocks(model: nn.Module, attr: str, layout: LoopLayout | None = None, *, repetitions: int = 2,
                step: Callable | None = None) -> LoopedStack:
    """Replaces ``model.<attr>`` (a ``ModuleList``) by a ``LoopedStack`` over the same block objects.  Parameter
    names change from ``<attr>.i.*`` to ``<attr>.blocks.i.*``; each block is still registered exactly once."""
    blocks = getattr(model, attr)
    stack = LoopedStack(blocks, layout or balanced_layout(len(blocks)), repetitions=repetitions, step=step)
    setattr(model, attr, stack)
    return stack
