"""Process-grid helpers: the teams of a data x tensor (or data x expert) parallel job.

Ranks are laid out row-major on a ``dp x inner`` grid: the ``inner`` consecutive ranks of a row form a tensor-
parallel (or expert-parallel) team, the ranks of a column (stride ``inner``) form a data-parallel team. Both are
strided sets, so they are plain OpenSHMEM teams (``team_split_strided``); the reference offers the same building
block and nothing above it (src/rocshmem.cpp:221-303).

    layout = ParallelLayout(inner=4)        # 8 ranks: two rows of four
    layout.inner_team                       # my row: all-gather -> GEMM, dispatch / combine ...
    layout.dp_team                          # my column: gradient all-reduce
"""
from __future__ import annotations

from typing import Optional

from .. import runtime as rt


class ParallelLayout:
    """The row (inner) and column (data-parallel) teams of this rank on a ``dp x inner`` grid; collective to create."""

    def __init__(self, inner: int, world: Optional[rt.Team] = None):
        self.world = world or rt.team_world()
        n, me = self.world.n_pes(), self.world.my_pe()
        if inner < 1 or n % inner:
            raise ValueError(f"the team size {n} is not a multiple of the inner dimension {inner}")
        self.inner, self.dp = inner, n // inner
        self.row, self.col = me // inner, me % inner
        # Splits are collective over the parent: every rank takes part in every split and keeps its own team.
        self.inner_team = None
        for r in range(self.dp):
            t = self.world.split_strided(r * inner, 1, inner)
            if r == self.row:
                self.inner_team = t
        self.dp_team = None
        for c in range(inner):
            t = self.world.split_strided(c, inner, self.dp)
            if c == self.col:
                self.dp_team = t

    def inner_rank(self) -> int:
        """My index inside the inner (tensor- or expert-parallel) team."""
        return self.col

    def dp_rank(self) -> int:
        """My index inside the data-parallel team."""
        return self.row

    def destroy(self) -> None:
        """Destroy both teams (collective)."""
        for t in (self.inner_team, self.dp_team):
            if t is not None and t.valid:
                t.destroy()
        self.inner_team = self.dp_team = None
