"""ARC grid DSL, executor and test-time ensembling.

Grids, the eight dihedral actions with their inverses, colour permutations, a closed
nine-instruction DSL (the dihedrals and ``recolor``), consistency of a program with
demonstration pairs, synthesis from a catalog, majority vote and the
augment -> execute -> undo ensemble, plus the ids the serving fork's test-time-training hook
loads. API parity with the reference ``arc/__init__.py`` (:39-293). The grid transforms
themselves are the C++ ones shared with the procedural generator
(``native.synth.arc``), so training data and the solver agree on what "rot90" means;
``default_catalog`` (all programs of at most two instructions) is an addition.
"""
from __future__ import annotations

from collections import Counter
from dataclasses import dataclass
from enum import Enum
from itertools import product

from .native import NativeError
from .native import synth as _synth

_A = _synth.arc

N_COLORS = 10
N_DIHEDRAL = 8
MIN_GRID_SIZE = 1
MAX_GRID_SIZE = 30
DIHEDRAL_NAMES: tuple[str, ...] = tuple(_A.DIHEDRALS)
_INVERSE = (0, 3, 2, 1, 4, 5, 6, 7)      # rot90 <-> rot270; everything else is an involution


class ArcError(ValueError):
    """A grid, program or sidecar id breaks an invariant."""


class OpKind(str, Enum):
    IDENTITY = "identity"
    ROT90 = "rot90"
    ROT180 = "rot180"
    ROT270 = "rot270"
    FLIP_H = "flip_h"
    FLIP_V = "flip_v"
    TRANSPOSE = "transpose"
    ANTI_TRANSPOSE = "anti_transpose"
    RECOLOR = "recolor"


@dataclass(frozen=True)
class Grid:
    cells: tuple


@dataclass(frozen=True)
class Pair:
    input: Grid
    output: Grid


@dataclass(frozen=True)
class Op:
    kind: OpKind
    src: int | None = None
    dst: int | None = None


@dataclass(frozen=True)
class Program:
    ops: tuple


@dataclass(frozen=True)
class SidecarHook:
    task_id: str
    lora_id: str


def _native(fn, *args):
    try:
        return fn(*args)
    except NativeError as e:
        raise ArcError(str(e)) from None


def make_grid(cells) -> Grid:
    rows = [list(r) for r in cells]
    for r in rows:
        for c in r:
            if isinstance(c, bool) or not isinstance(c, int) or not 0 <= c < N_COLORS:
                raise ArcError(f"color {c} outside 0..{N_COLORS}")
    checked = _native(_A.validate_grid, rows)
    return Grid(tuple(tuple(int(c) for c in r) for r in checked))


def _rows(grid: Grid) -> list:
    return [list(r) for r in grid.cells]


def _index(index) -> int:
    if isinstance(index, bool) or not isinstance(index, int) or not 0 <= index < N_DIHEDRAL:
        raise ArcError(f"dihedral index {index} out of range")
    return index


def apply_dihedral(grid: Grid, index: int) -> Grid:
    return make_grid(_native(_A.apply_dihedral, _rows(grid), _index(index)))


def inverse_dihedral(index: int) -> int:
    return _INVERSE[_index(index)]


def apply_color_perm(grid: Grid, perm) -> Grid:
    p = [int(x) for x in perm]
    if sorted(p) != list(range(N_COLORS)):
        raise ArcError("color permutation is not a permutation of 0..10")
    return make_grid(_native(_A.apply_color_perm, _rows(grid), p))


def _step(op: Op, grid: Grid) -> Grid:
    if op.kind is OpKind.RECOLOR:
        if op.src is None or op.dst is None:
            raise ArcError("recolor requires src and dst")
        if op.src not in range(N_COLORS) or op.dst not in range(N_COLORS):
            raise ArcError("recolor src/dst out of range")
        return Grid(tuple(tuple(op.dst if c == op.src else c for c in r) for r in grid.cells))
    try:
        return apply_dihedral(grid, DIHEDRAL_NAMES.index(OpKind(op.kind).value))
    except ValueError as e:
        raise ArcError(f"unknown op kind {op.kind}") from e


def execute(program: Program, grid: Grid) -> Grid:
    cur = make_grid(_rows(grid))
    for op in program.ops:
        cur = _step(op, cur)
    return cur


def consistent(program: Program, train) -> bool:
    if not train:
        raise ArcError("empty train")
    return all(execute(program, p.input).cells == make_grid(_rows(p.output)).cells for p in train)


def synthesize(train, catalog):
    if not train:
        raise ArcError("empty train")
    if not catalog:
        raise ArcError("empty catalog")
    return next((prog for prog in catalog if consistent(prog, train)), None)


def default_catalog(max_ops: int = 2) -> tuple:
    """Every program of at most ``max_ops`` instructions, shortest first (identity, the 7 other
    dihedrals, the 90 recolours, then their compositions)."""
    atoms = [Op(OpKind(n)) for n in DIHEDRAL_NAMES[1:]]
    atoms += [Op(OpKind.RECOLOR, s, d) for s in range(N_COLORS) for d in range(N_COLORS) if s != d]
    progs = [Program(())]
    for n in range(1, max_ops + 1):
        progs += [Program(tuple(c)) for c in product(atoms, repeat=n)]
    return tuple(progs)


def vote(grids) -> Grid:
    if not grids:
        raise ArcError("empty grids")
    counts = Counter(g.cells for g in grids)          # insertion order = first appearance
    best = max(counts, key=lambda k: counts[k])       # max keeps the earliest among ties
    return Grid(best)


def ensemble_predict(program: Program, test_input: Grid, dihedrals) -> Grid:
    if not dihedrals:
        raise ArcError("empty dihedrals")
    outs = [apply_dihedral(execute(program, apply_dihedral(test_input, k)), inverse_dihedral(k)) for k in dihedrals]
    return vote(tuple(outs))


def sidecar_hook(task_id: str, lora_id: str) -> SidecarHook:
    if not task_id or not lora_id:
        raise ArcError("task_id and lora_id must be non-empty")
    return SidecarHook(task_id, lora_id)
