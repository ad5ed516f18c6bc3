"""Teams: integer handles for strided sub-groups of the job, with the calling convention of the
reference's ``_nvshmem_team_*`` bindings (src/pybind/ths_op.cc:227-300, thin wrappers over
``nvshmem_team_split_strided`` / ``split_2d`` / ``translate_pe`` / ``n_pes`` / ``my_pe``).

There is no NVSHMEM here: a team is a record (start, stride, size in world ranks) plus a torch
process group created for its members, so that the ops of this library, which take process
groups, can run on a team (``team_group(team)``). Team 0 is the world. As with NVSHMEM, a split is
collective over the parent team: every member calls it with the same arguments; ranks outside the
new team get ``TEAM_INVALID``.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

import torch.distributed as dist

TEAM_WORLD = 0
TEAM_INVALID = -1


@dataclasses.dataclass
class TeamConfig:
    """Opaque to callers in the reference (``nvshmem_team_config_t``); here it names the geometry."""
    start: int
    stride: int
    size: int


@dataclasses.dataclass
class _Team:
    cfg: TeamConfig
    group: Optional[object]


_TEAMS: Dict[int, _Team] = {}
_NEXT = [1]


def _world() -> _Team:
    if TEAM_WORLD not in _TEAMS:
        _TEAMS[TEAM_WORLD] = _Team(TeamConfig(0, 1, dist.get_world_size()), dist.group.WORLD)
    return _TEAMS[TEAM_WORLD]


def _get(team: int) -> _Team:
    if team == TEAM_WORLD:
        return _world()
    if team not in _TEAMS:
        raise ValueError(f"unknown team {team}")
    return _TEAMS[team]


def _members(cfg: TeamConfig):
    return [cfg.start + i * cfg.stride for i in range(cfg.size)]


def team_group(team: int):
    """The process group of a team (pass it to the ops)."""
    return _get(team).group


def _nvshmem_team_npes(team: int) -> int:
    return _get(team).cfg.size


def _nvshmem_team_my_pe(team: int) -> int:
    cfg = _get(team).cfg
    me = dist.get_rank()
    off = me - cfg.start
    if off < 0 or off % cfg.stride or off // cfg.stride >= cfg.size:
        return -1
    return off // cfg.stride


def _nvshmem_team_get_config(team: int) -> TeamConfig:
    return dataclasses.replace(_get(team).cfg)


def _nvshmem_team_translate_pe(src_team: int, src_pe: int, dest_team: int) -> int:
    """PE number in ``dest_team`` of the process that is ``src_pe`` in ``src_team`` (-1 if it is
    not a member)."""
    s, d = _get(src_team).cfg, _get(dest_team).cfg
    if src_pe < 0 or src_pe >= s.size:
        return -1
    world_rank = s.start + src_pe * s.stride
    off = world_rank - d.start
    if off < 0 or off % d.stride or off // d.stride >= d.size:
        return -1
    return off // d.stride


def _nvshmem_team_split_strided(parent_team: int, PE_start: int, PE_stride: int, PE_size: int,
                                config: Optional[TeamConfig] = None, config_mask: int = 0) -> int:
    """New team of the parent's PEs PE_start, PE_start + PE_stride, ... (PE_size of them).
    Collective over the job (``dist.new_group`` is); every rank gets the same handle number, ranks
    outside the team get ``TEAM_INVALID`` back."""
    p = _get(parent_team).cfg
    if PE_size < 1 or PE_stride < 1 or PE_start < 0 or PE_start + (PE_size - 1) * PE_stride >= p.size:
        raise ValueError("team geometry outside the parent team")
    cfg = TeamConfig(p.start + PE_start * p.stride, p.stride * PE_stride, PE_size)
    group = dist.new_group(ranks=_members(cfg))
    handle = _NEXT[0]
    _NEXT[0] += 1
    _TEAMS[handle] = _Team(cfg, group)
    return handle if dist.get_rank() in _members(cfg) else TEAM_INVALID


def _nvshmem_team_split_2d(parent_team: int, xrange: int, xaxis_config: Optional[TeamConfig] = None,
                           xaxis_mask: int = 0, yaxis_config: Optional[TeamConfig] = None,
                           yaxis_mask: int = 0) -> Tuple[int, int]:
    """The parent's PEs as a grid with ``xrange`` columns: returns (team of my row, team of my column)."""
    p = _get(parent_team).cfg
    if xrange < 1:
        raise ValueError("xrange")
    ny = -(-p.size // xrange)
    me = _nvshmem_team_my_pe(parent_team)
    mine_x = mine_y = TEAM_INVALID
    for y in range(ny):                       # every rank creates every team: new_group is collective
        n = min(xrange, p.size - y * xrange)
        t = _nvshmem_team_split_strided(parent_team, y * xrange, 1, n)
        if me >= 0 and me // xrange == y:
            mine_x = t
    for x in range(min(xrange, p.size)):
        n = len(range(x, p.size, xrange))
        t = _nvshmem_team_split_strided(parent_team, x, xrange, n)
        if me >= 0 and me % xrange == x:
            mine_y = t
    return mine_x, mine_y


def _nvshmem_team_destroy(team: int) -> None:
    if team in (TEAM_WORLD, TEAM_INVALID):
        return
    t = _TEAMS.pop(team, None)
    if t is not None and t.group is not None and dist.get_rank() in _members(t.cfg):
        dist.destroy_process_group(t.group)
