"""Behaviour list of the ARC grid DSL (``prometheus_b200.arc``; reference tests/test_arc.py and
arc/__init__.py:39-293): grid validation, the eight dihedral actions against NumPy, inverses,
colour permutations, program execution, consistency, synthesis order, majority vote with
earliest-wins ties, the augment-execute-undo ensemble and the sidecar ids."""
import dataclasses
import itertools
import random

import numpy as np
import pytest

from prometheus_b200 import arc as A

G23 = [[1, 2, 3], [4, 5, 6]]
NP_DIHEDRAL = [lambda a: a, lambda a: np.rot90(a, -1), lambda a: np.rot90(a, 2), lambda a: np.rot90(a, 1),
               lambda a: a[:, ::-1], lambda a: a[::-1, :], lambda a: a.T, lambda a: np.rot90(a, 2).T]


def cells(a):
    return tuple(tuple(int(c) for c in row) for row in np.asarray(a))


# ------------------------------------------------------------------------------ constants / types
def test_constants_names_and_kinds():
    assert (A.N_COLORS, A.N_DIHEDRAL, A.MIN_GRID_SIZE, A.MAX_GRID_SIZE) == (10, 8, 1, 30)
    assert A.DIHEDRAL_NAMES == ("identity", "rot90", "rot180", "rot270", "flip_h", "flip_v", "transpose", "anti_transpose")
    assert [k.value for k in A.OpKind] == list(A.DIHEDRAL_NAMES) + ["recolor"]
    assert issubclass(A.ArcError, ValueError)
    g = A.make_grid(G23)
    for obj in (g, A.Pair(g, g), A.Op(A.OpKind.ROT90), A.Program(()), A.SidecarHook("t", "l")):
        with pytest.raises(dataclasses.FrozenInstanceError):
            setattr(obj, dataclasses.fields(obj)[0].name, None)


# ------------------------------------------------------------------------------ grids
def test_make_grid_freezes_and_copies():
    src = [[1, 2], [3, 4]]
    g = A.make_grid(src)
    src[0][0] = 9
    assert g.cells == ((1, 2), (3, 4)) and isinstance(g.cells, tuple) and isinstance(g.cells[0], tuple)
    assert A.make_grid([[0]]).cells == ((0,),) and A.make_grid([[9]]).cells == ((9,),)
    big = A.make_grid([[0] * 30 for _ in range(30)])
    assert len(big.cells) == 30 and len(big.cells[0]) == 30
    assert A.make_grid(((1, 2), (3, 4))) == A.make_grid([[1, 2], [3, 4]])


@pytest.mark.parametrize("bad", [[], [[]], [[1, 2], [3]], [[0] * 31], [[0]] * 31, [[10]], [[-1]], [[1.5]], [[True]], [["1"]]])
def test_make_grid_rejects(bad):
    with pytest.raises(A.ArcError):
        A.make_grid(bad)


# ------------------------------------------------------------------------------ dihedral group
@pytest.mark.parametrize("index", range(8))
def test_dihedral_actions_match_numpy(index):
    rng = np.random.default_rng(index)
    for h, w in ((2, 3), (1, 1), (1, 5), (4, 4), (3, 7)):
        a = rng.integers(0, 10, size=(h, w))
        got = A.apply_dihedral(A.make_grid(a.tolist()), index)
        assert got.cells == cells(NP_DIHEDRAL[index](a))
        if index in (1, 3, 6, 7):
            assert (len(got.cells), len(got.cells[0])) == (w, h)                       # height and width swap
    assert A.apply_dihedral(A.make_grid([[7]]), index).cells == ((7,),)


def test_rot90_is_clockwise():
    assert A.apply_dihedral(A.make_grid(G23), 1).cells == ((4, 1), (5, 2), (6, 3))
    assert A.apply_dihedral(A.make_grid(G23), 4).cells == ((3, 2, 1), (6, 5, 4))       # flip_h mirrors left-right
    assert A.apply_dihedral(A.make_grid(G23), 5).cells == ((4, 5, 6), (1, 2, 3))


def test_inverse_table():
    assert [A.inverse_dihedral(k) for k in range(8)] == [0, 3, 2, 1, 4, 5, 6, 7]
    assert all(A.inverse_dihedral(A.inverse_dihedral(k)) == k for k in range(8))
    rng = np.random.default_rng(0)
    for k in range(8):
        g = A.make_grid(rng.integers(0, 10, size=(3, 5)).tolist())
        assert A.apply_dihedral(A.apply_dihedral(g, k), A.inverse_dihedral(k)) == g


@pytest.mark.parametrize("index", [-1, 8, 100, 1.0, True, None, "1"])
def test_dihedral_index_out_of_range(index):
    g = A.make_grid(G23)
    with pytest.raises(A.ArcError):
        A.apply_dihedral(g, index)
    with pytest.raises(A.ArcError):
        A.inverse_dihedral(index)


# ------------------------------------------------------------------------------ colour permutations
def test_colour_permutations():
    g = A.make_grid([[0, 1, 2], [9, 0, 1]])
    assert A.apply_color_perm(g, range(10)) == g
    swap = [1, 0] + list(range(2, 10))
    assert A.apply_color_perm(g, swap).cells == ((1, 0, 2), (9, 1, 0))                  # colour 0 is not special
    cycle = [(c + 1) % 10 for c in range(10)]
    assert A.apply_color_perm(g, cycle).cells == ((1, 2, 3), (0, 1, 2))
    inverse = [cycle.index(c) for c in range(10)]
    assert A.apply_color_perm(A.apply_color_perm(g, cycle), inverse) == g
    for bad in (list(range(9)), list(range(11)), [0] * 10, [0, 1, 2, 3, 4, 5, 6, 7, 8, 10], [1] + list(range(1, 10))):
        with pytest.raises(A.ArcError):
            A.apply_color_perm(g, bad)


# ------------------------------------------------------------------------------ programs
def test_execution():
    g = A.make_grid([[1, 2], [1, 0]])
    assert A.execute(A.Program(()), g) == g
    assert A.execute(A.Program((A.Op(A.OpKind.RECOLOR, 1, 2),)), g).cells == ((2, 2), (2, 0))
    assert A.execute(A.Program((A.Op(A.OpKind.RECOLOR, 3, 3),)), g) == g
    assert A.execute(A.Program((A.Op(A.OpKind.ROT90, 5, 6),)), g) == A.apply_dihedral(g, 1)         # src / dst ignored
    two = A.Program((A.Op(A.OpKind.RECOLOR, 1, 2), A.Op(A.OpKind.RECOLOR, 2, 3)))                   # left to right
    assert A.execute(two, g).cells == ((3, 3), (3, 0))
    back = A.Program((A.Op(A.OpKind.RECOLOR, 2, 3), A.Op(A.OpKind.RECOLOR, 1, 2)))
    assert A.execute(back, g).cells == ((2, 3), (2, 0))
    assert A.execute(A.Program((A.Op(A.OpKind.ROT90), A.Op(A.OpKind.ROT270))), g) == g
    order = A.Program((A.Op(A.OpKind.ROT90), A.Op(A.OpKind.FLIP_H)))
    assert A.execute(order, A.make_grid(G23)).cells == cells(np.rot90(np.array(G23), -1)[:, ::-1])
    for op in (A.Op(A.OpKind.RECOLOR), A.Op(A.OpKind.RECOLOR, 1), A.Op(A.OpKind.RECOLOR, None, 1), A.Op(A.OpKind.RECOLOR, -1, 2),
               A.Op(A.OpKind.RECOLOR, 1, 10), A.Op("spin")):
        with pytest.raises(A.ArcError):
            A.execute(A.Program((op,)), g)


def test_consistency_and_synthesis_order():
    g1, g2 = A.make_grid(G23), A.make_grid([[7, 8], [9, 0]])
    flip = A.Program((A.Op(A.OpKind.FLIP_H),))
    train = [A.Pair(g, A.apply_dihedral(g, 4)) for g in (g1, g2)]
    assert A.consistent(flip, train) and not A.consistent(A.Program(()), train)
    assert not A.consistent(flip, train + [A.Pair(g1, g1)])
    catalog = [A.Program((A.Op(A.OpKind(n)),)) for n in A.DIHEDRAL_NAMES]
    assert A.synthesize(train, catalog) == flip
    assert A.synthesize([A.Pair(g1, A.make_grid([[0]]))], catalog) is None
    sym = A.make_grid([[1, 1], [1, 1]])                                                # every dihedral fits: the first wins
    assert A.synthesize([A.Pair(sym, sym)], catalog) == catalog[0]
    assert A.synthesize([A.Pair(sym, sym)], catalog[::-1]) == catalog[-1]
    for call in (lambda: A.consistent(flip, []), lambda: A.synthesize([], catalog), lambda: A.synthesize(train, [])):
        with pytest.raises(A.ArcError):
            call()
    cat = A.default_catalog(1)
    assert cat[0] == A.Program(()) and len(cat) == 1 + 7 + 90 and len(A.default_catalog(2)) == 98 + 97 * 97
    recol = [A.Pair(g1, A.execute(A.Program((A.Op(A.OpKind.RECOLOR, 1, 9),)), g1))]
    assert A.synthesize(recol, cat) == A.Program((A.Op(A.OpKind.RECOLOR, 1, 9),))


# ------------------------------------------------------------------------------ vote / ensemble
def test_vote():
    a, b, c = A.make_grid([[1]]), A.make_grid([[2]]), A.make_grid([[1, 1]])
    assert A.vote((a, a, b)) == a and A.vote((a, b)) == a and A.vote((b, a)) == b          # a tie keeps the earliest
    assert A.vote((a, b, b)) == b                                                          # a later majority overtakes
    assert A.vote((a, c, c, a, a)) == a and A.vote((c, a)) == c                            # other shapes are other candidates
    with pytest.raises(A.ArcError):
        A.vote(())
    rng = random.Random(0)
    pool = [a, b, c, A.make_grid([[3]])]
    for _ in range(100):
        picks = [rng.choice(pool) for _ in range(rng.randint(1, 9))]
        counts = {}
        for g in picks:
            counts[g] = counts.get(g, 0) + 1
        top = max(counts.values())
        assert A.vote(tuple(picks)) == next(g for g in picks if counts[g] == top)


def test_ensemble_augments_executes_and_undoes():
    g = A.make_grid(G23)
    ident = A.Program(())
    assert A.ensemble_predict(ident, g, tuple(range(8))) == g and A.ensemble_predict(ident, g, (0,)) == g
    recolor = A.Program((A.Op(A.OpKind.RECOLOR, 1, 9),))                                   # commutes with every dihedral
    assert A.ensemble_predict(recolor, g, tuple(range(8))) == A.execute(recolor, g)
    rot = A.Program((A.Op(A.OpKind.ROT90),))                                               # rotations commute with rotations
    assert A.ensemble_predict(rot, g, (0, 1, 2, 3)) == A.apply_dihedral(g, 1)
    for bad in ((), (8,), (0, -1), (0, 1.0)):
        with pytest.raises(A.ArcError):
            A.ensemble_predict(ident, g, bad)


def test_sidecar_ids():
    assert A.sidecar_hook("task-1", "lora-9") == A.SidecarHook("task-1", "lora-9")
    for t, l in (("", "l"), ("t", ""), ("", "")):
        with pytest.raises(A.ArcError):
            A.sidecar_hook(t, l)


def test_group_table_closes():
    g = A.make_grid([[1, 2, 3], [4, 5, 6], [7, 8, 0]])
    images = [A.apply_dihedral(g, k) for k in range(8)]
    assert len(set(images)) == 8
    for i, j in itertools.product(range(8), repeat=2):
        assert A.apply_dihedral(A.apply_dihedral(g, i), j) in images
