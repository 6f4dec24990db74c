"""Template builders for the four supported algorithms: PPO, GRPO, DPO and PPO with a shared
actor-critic trunk.

Each template is written as a small table (vertices with read/write container names, data edges,
publication edges) that one generic routine turns into an ``RPEG``. Vertex ids, container names
and sizes, edge sets and default staleness equal the reference's builders
(RPEG/ir/ppo.py:17-114, grpo.py:17-108, dpo.py:63-166, ac_share.py:29-118) so plans are
interchangeable: activations are 2-byte elements sized from (B, K, S, T), weights are
``n_params`` 2-byte elements.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

from ..analytic.models import ModelSuite
from ..analytic.workload import Workload
from ..core.types import Container, EdgeKind, Model, OperatorKind, Role, TemplateEdge, TemplateVertex
from .rpeg import RPEG

G, I, T_ = Role.GENERATION, Role.INFERENCE, Role.TRAINING

# (vertex id, role, model, reads, writes)
_PPO = dict(
    vertices=[
        ("g_pi", G, Model.ACTOR, ("W_pi", "prompts"), ("completions", "log_pi")),
        ("i_ref", I, Model.REFERENCE, ("W_ref", "completions"), ("log_ref",)),
        ("i_R", I, Model.REWARD, ("W_R", "completions"), ("rewards",)),
        ("i_V", I, Model.CRITIC, ("W_V", "completions"), ("values",)),
        ("t_pi", T_, Model.ACTOR, ("W_pi", "completions", "log_pi", "log_ref", "rewards", "values"), ("W_pi",)),
        ("t_V", T_, Model.CRITIC, ("W_V", "completions", "log_ref", "rewards", "values"), ("W_V",)),
    ],
    data=[("g_pi", "i_ref", "completions"), ("g_pi", "i_R", "completions"), ("g_pi", "i_V", "completions"),
          ("i_ref", "t_pi", "log_ref"), ("i_ref", "t_V", "log_ref"), ("i_R", "t_pi", "rewards"),
          ("i_V", "t_pi", "values"), ("i_R", "t_V", "rewards"), ("i_V", "t_V", "values")],
    pub=[("t_pi", "g_pi", "W_pi"), ("t_V", "i_V", "W_V")],
    containers=("completions", "log_pi", "log_ref", "rewards", "values", "W_pi", "W_V", "W_ref", "W_R"),
    inputs=("prompts", "W_ref", "W_R"),
    trainable=(Model.ACTOR, Model.CRITIC),
)

_GRPO = dict(
    vertices=[
        ("g_pi", G, Model.ACTOR, ("W_pi", "prompts"), ("completions", "log_pi")),
        ("i_ref", I, Model.REFERENCE, ("W_ref", "completions"), ("log_ref",)),
        ("i_R", I, Model.REWARD, ("W_R", "completions"), ("rewards",)),
        ("t_pi", T_, Model.ACTOR, ("W_pi", "completions", "log_pi", "log_ref", "rewards"), ("W_pi",)),
    ],
    data=[("g_pi", "i_ref", "completions"), ("g_pi", "i_R", "completions"),
          ("i_ref", "t_pi", "log_ref"), ("i_R", "t_pi", "rewards")],
    pub=[("t_pi", "g_pi", "W_pi")],
    containers=("completions", "log_pi", "log_ref", "rewards", "W_pi", "W_ref", "W_R"),
    inputs=("prompts", "W_ref", "W_R"),
    trainable=(Model.ACTOR,),
)

_DPO = dict(
    vertices=[
        ("i_pi", I, Model.ACTOR, ("W_pi", "X_pref"), ("log_pi",)),
        ("i_ref", I, Model.REFERENCE, ("W_ref", "X_pref"), ("log_ref",)),
        ("t_pi", T_, Model.ACTOR, ("W_pi", "X_pref", "log_pi", "log_ref"), ("W_pi",)),
    ],
    data=[("i_pi", "t_pi", "log_pi"), ("i_ref", "t_pi", "log_ref")],
    pub=[("t_pi", "i_pi", "W_pi")],
    containers=("log_pi", "log_ref", "W_pi", "W_ref"),
    inputs=("X_pref", "W_ref"),
    trainable=(Model.ACTOR,),
)

_AC = dict(
    vertices=[
        ("g_ac", G, Model.AC_SHARE, ("W_AC", "prompts"), ("completions", "log_ac")),
        ("i_ref", I, Model.REFERENCE, ("W_ref", "completions"), ("log_ref",)),
        ("i_R", I, Model.REWARD, ("W_R", "completions"), ("rewards",)),
        ("i_ac", I, Model.AC_SHARE, ("W_AC", "completions"), ("values",)),
        ("t_ac", T_, Model.AC_SHARE, ("W_AC", "completions", "log_ac", "log_ref", "rewards", "values"), ("W_AC",)),
    ],
    data=[("g_ac", "i_ref", "completions"), ("g_ac", "i_R", "completions"), ("g_ac", "i_ac", "completions"),
          ("i_ref", "t_ac", "log_ref"), ("i_R", "t_ac", "rewards"), ("i_ac", "t_ac", "values")],
    pub=[("t_ac", "g_ac", "W_AC"), ("t_ac", "i_ac", "W_AC")],
    containers=("completions", "log_ac", "log_ref", "rewards", "values", "W_AC", "W_ref", "W_R"),
    inputs=("prompts", "W_ref", "W_R"),
    trainable=(Model.AC_SHARE,),
)

_WEIGHT_MODEL = {"W_pi": Model.ACTOR, "W_V": Model.CRITIC, "W_ref": Model.REFERENCE, "W_R": Model.REWARD,
                 "W_AC": Model.AC_SHARE}


def _container_table(suite: ModelSuite, w: Workload, pairwise: bool) -> Dict[str, Container]:
    B, K, S, T = w.B, w.K, w.S, w.T
    sizes = {
        "prompts": B * S,
        "completions": B * K * (S + T),
        "log_pi": B * 2 * T if pairwise else B * K * T,
        "log_ac": B * K * T,
        "log_ref": B * 2 * T if pairwise else B * K * T,
        "rewards": B * K,
        "values": B * K * T,
        "X_pref": B * 2 * (S + T),
    }
    table = {name: Container(name, count, 2) for name, count in sizes.items()}
    for name, model in _WEIGHT_MODEL.items():
        if model in suite.specs:
            table[name] = Container(name, suite.n_params(model), 2)
    return table


def _instantiate(spec: dict, suite: ModelSuite, workload: Workload, tau: Optional[Dict[Model, int]],
                 pairwise: bool, verbose: bool) -> RPEG:
    table = _container_table(suite, workload, pairwise)
    pick = lambda names: tuple(table[n] for n in names)  # noqa: E731
    verts = {vid: TemplateVertex(vid, OperatorKind(role, model, pick(rd), pick(wr)))
             for vid, role, model, rd, wr in spec["vertices"]}
    mk = lambda rows, kind: tuple(TemplateEdge(verts[s], verts[d], table[c], kind) for s, d, c in rows)  # noqa: E731
    trainable = set(spec["trainable"])
    if tau is None:
        tau = {m: 0 for m in trainable}
    rpeg = RPEG(tuple(verts.values()), mk(spec["data"], EdgeKind.DATA), mk(spec["pub"], EdgeKind.PUB),
                pick(spec["containers"]), pick(spec["inputs"]), (), dict(tau), trainable)
    rpeg.well_formed(verbose)
    return rpeg


def build_PPO_RPEG(suite, workload, tau=None, verbose=False) -> RPEG:
    return _instantiate(_PPO, suite, workload, tau, False, verbose)


def build_GRPO_RPEG(suite, workload, tau=None, verbose=False) -> RPEG:
    return _instantiate(_GRPO, suite, workload, tau, False, verbose)


def build_DPO_RPEG(suite, workload, tau=None, verbose=False) -> RPEG:
    return _instantiate(_DPO, suite, workload, tau, True, verbose)


def build_AC_share_RPEG(suite, workload, tau=None, verbose=False) -> RPEG:
    return _instantiate(_AC, suite, workload, tau, False, verbose)


def is_AC_share_applicable(rpeg: RPEG) -> bool:
    """Sharing a trunk needs both an actor and a critic to train."""
    return Model.ACTOR in rpeg.trainable and Model.CRITIC in rpeg.trainable


BUILDERS = {"ppo": build_PPO_RPEG, "grpo": build_GRPO_RPEG, "dpo": build_DPO_RPEG, "ac_share": build_AC_share_RPEG}


def build_rpeg(algorithm: str, suite, workload, tau=None, verbose=False) -> RPEG:
    builder = BUILDERS.get(algorithm.lower())
    if builder is None:
        raise ValueError(f"unknown algorithm {algorithm!r}; expected one of {sorted(BUILDERS)}")
    return builder(suite, workload, tau, verbose)
