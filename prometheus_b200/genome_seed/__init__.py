"""Seed genome of the research lab: role descriptions, the seed program, tool and skill notes
(Markdown next to this file) and their loader.

API parity with the reference's ``harness/genome-seed/genome_seed.py`` (:16-131): ``ROLES``,
``load_seed``, ``role_names``, ``require_roles``, ``GenomeSeed`` with ``roles`` / ``programs`` /
``tools`` / ``skills``. ``instructions_for`` composes what a spawned agent of a role is given
(its role text followed by every program), the text the lab kernel prefixes with its invariant.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

SEED_DIR = Path(__file__).resolve().parent
ROLES = ("director", "researcher", "implementer", "reviewer", "tester")


class GenomeError(ValueError):
    """The seed tree is missing or lacks a required role."""


@dataclass(frozen=True)
class Entry:
    name: str
    body: str


Role = Program = ToolSpec = Skill = Entry


@dataclass(frozen=True)
class GenomeSeed:
    roles: tuple
    programs: tuple
    tools: tuple
    skills: tuple
    root: Path


def seed_root() -> Path:
    return SEED_DIR


def _markdown(directory: Path) -> tuple:
    if not directory.is_dir():
        return ()
    return tuple(Entry(p.stem, p.read_text(encoding="utf-8"))
                 for p in sorted(directory.iterdir(), key=lambda p: p.name) if p.is_file() and p.suffix == ".md")


def load_seed(root: Path | None = None) -> GenomeSeed:
    root = Path(SEED_DIR if root is None else root).resolve()
    if not root.is_dir():
        raise GenomeError(f"seed root is not a directory: {root}")
    roles = _markdown(root / "roles")
    rank = {n: i for i, n in enumerate(ROLES)}
    roles = tuple(sorted(roles, key=lambda r: (rank.get(r.name, len(ROLES)), r.name)))
    seed = GenomeSeed(roles, _markdown(root / "programs"), _markdown(root / "tools"), _markdown(root / "skills"), root)
    require_roles(seed)
    return seed


def role_names(seed: GenomeSeed) -> tuple:
    return tuple(r.name for r in seed.roles)


def require_roles(seed: GenomeSeed) -> None:
    have = {r.name for r in seed.roles}
    missing = [n for n in ROLES if n not in have]
    if missing:
        raise GenomeError("missing required role(s): " + ", ".join(missing))


def instructions_for(seed: GenomeSeed, role: str) -> str:
    by_name = {r.name: r for r in seed.roles}
    if role not in by_name:
        raise GenomeError(f"unknown role {role}")
    return "\n\n".join([by_name[role].body.strip()] + [p.body.strip() for p in seed.programs])
