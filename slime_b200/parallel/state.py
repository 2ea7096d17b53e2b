"""Process-group topology for TP / CP / EP / DP / PP.

Replaces the ``mpu`` rank/group queries the reference takes from Megatron-core
(slime/backends/megatron_utils/initialize.py:33-53). Rank order is
``tp-cp-ep-dp-pp`` (TP fastest), i.e. TP peers are adjacent GPUs, which on an
NVSwitch box makes no bandwidth difference but keeps rank<->GPU maps readable.

Without an initialised ``torch.distributed`` every size is 1 and every rank 0,
so single-process CPU code can call the queries unconditionally.
"""

from __future__ import annotations

import dataclasses
import itertools
from typing import Any

import torch
import torch.distributed as dist


@dataclasses.dataclass
class _Axis:
    size: int = 1
    rank: int = 0
    group: Any = None
    ranks: list[int] = dataclasses.field(default_factory=lambda: [0])
    gloo_group: Any = None


class ParallelState:
    """Holds one `_Axis` per parallel dimension plus combined groups."""

    AXES = ("tp", "cp", "dp", "pp", "ep", "etp", "edp", "dp_cp", "tp_cp", "mp", "embd")

    def __init__(self):
        self.reset()

    def reset(self):
        self.initialized = False
        self.world_size = 1
        self.rank = 0
        self.virtual_pp_size: int | None = None
        self.virtual_pp_rank: int | None = None
        for a in self.AXES:
            setattr(self, a, _Axis())

    # -- layout helpers -------------------------------------------------
    @staticmethod
    def decompose(rank: int, sizes: dict[str, int], order: tuple[str, ...]) -> dict[str, int]:
        """Coordinates of ``rank`` for a mixed-radix layout with ``order[0]`` fastest."""
        out = {}
        for name in order:
            out[name] = rank % sizes[name]
            rank //= sizes[name]
        return out

    @staticmethod
    def compose(coord: dict[str, int], sizes: dict[str, int], order: tuple[str, ...]) -> int:
        rank, stride = 0, 1
        for name in order:
            rank += coord[name] * stride
            stride *= sizes[name]
        return rank

    @classmethod
    def groups_along(cls, axes: tuple[str, ...], sizes: dict[str, int], order: tuple[str, ...]) -> list[list[int]]:
        """All rank lists obtained by varying ``axes`` and fixing the others."""
        var = [a for a in order if a in axes]
        fixed = [a for a in order if a not in axes]
        out = []
        for fv in itertools.product(*[range(sizes[a]) for a in fixed]):
            base = dict(zip(fixed, fv))
            members = []
            for vv in itertools.product(*[range(sizes[a]) for a in var]):
                members.append(cls.compose({**base, **dict(zip(var, vv))}, sizes, order))
            out.append(sorted(members))
        out.sort()
        return out


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def _make_groups(rank_lists: list[list[int]], my_rank: int, backend=None, with_gloo=False, timeout=None) -> _Axis:
    axis = _Axis()
    for ranks in rank_lists:
        kwargs = {}
        if timeout is not None:
            kwargs["timeout"] = timeout
        g = dist.new_group(ranks, backend=backend, **kwargs)
        gg = dist.new_group(ranks, backend="gloo", **kwargs) if with_gloo else None
        if my_rank in ranks:
            axis = _Axis(size=len(ranks), rank=ranks.index(my_rank), group=g, ranks=list(ranks), gloo_group=gg)
    return axis


def initialize_model_parallel(
    tensor_model_parallel_size: int = 1,
    pipeline_model_parallel_size: int = 1,
    virtual_pipeline_model_parallel_size: int | None = None,
    context_parallel_size: int = 1,
    expert_model_parallel_size: int = 1,
    expert_tensor_parallel_size: int | None = None,
    backend: str | None = None,
    timeout=None,
) -> ParallelState:
    """Create every process group. Must be called by all ranks in the same order."""
    st = _STATE
    st.reset()
    st.layout_args = dict(
        tensor_model_parallel_size=tensor_model_parallel_size, pipeline_model_parallel_size=pipeline_model_parallel_size,
        virtual_pipeline_model_parallel_size=virtual_pipeline_model_parallel_size, context_parallel_size=context_parallel_size,
        expert_model_parallel_size=expert_model_parallel_size, expert_tensor_parallel_size=expert_tensor_parallel_size,
        backend=backend, timeout=timeout,
    )  # fmt: skip
    if not dist.is_available() or not dist.is_initialized():
        assert (
            tensor_model_parallel_size * pipeline_model_parallel_size * context_parallel_size == 1
        ), "model parallelism needs torch.distributed to be initialised"
        st.initialized = True
        st.virtual_pp_size = virtual_pipeline_model_parallel_size
        return st

    world, rank = dist.get_world_size(), dist.get_rank()
    tp, pp, cp, ep = (
        tensor_model_parallel_size,
        pipeline_model_parallel_size,
        context_parallel_size,
        expert_model_parallel_size,
    )
    etp = tp if expert_tensor_parallel_size is None else expert_tensor_parallel_size
    assert world % (tp * pp * cp) == 0, f"world {world} not divisible by tp*pp*cp={tp * pp * cp}"
    dp = world // (tp * pp * cp)
    st.world_size, st.rank = world, rank

    # dense layout
    sizes = {"tp": tp, "cp": cp, "dp": dp, "pp": pp}
    order = ("tp", "cp", "dp", "pp")
    ga = lambda axes: ParallelState.groups_along(axes, sizes, order)  # noqa: E731
    st.tp = _make_groups(ga(("tp",)), rank, backend, timeout=timeout)
    st.cp = _make_groups(ga(("cp",)), rank, backend, timeout=timeout)
    st.dp = _make_groups(ga(("dp",)), rank, backend, with_gloo=True, timeout=timeout)
    st.pp = _make_groups(ga(("pp",)), rank, backend, timeout=timeout)
    st.dp_cp = _make_groups(ga(("dp", "cp")), rank, backend, with_gloo=True, timeout=timeout)
    st.tp_cp = _make_groups(ga(("tp", "cp")), rank, backend, timeout=timeout)
    st.mp = _make_groups(ga(("tp", "pp")), rank, backend, timeout=timeout)

    # expert layout: the tp*cp*dp ranks of one pipeline stage are re-factored as etp * ep * edp
    per_stage = tp * cp * dp
    assert per_stage % (etp * ep) == 0, f"tp*cp*dp={per_stage} not divisible by etp*ep={etp * ep}"
    edp = per_stage // (etp * ep)
    esizes = {"etp": etp, "ep": ep, "edp": edp, "pp": pp}
    eorder = ("etp", "ep", "edp", "pp")
    ega = lambda axes: ParallelState.groups_along(axes, esizes, eorder)  # noqa: E731
    st.etp = _make_groups(ega(("etp",)), rank, backend, timeout=timeout)
    st.ep = _make_groups(ega(("ep",)), rank, backend, timeout=timeout)
    st.edp = _make_groups(ega(("edp",)), rank, backend, with_gloo=True, timeout=timeout)

    # embedding group: first and last pipeline stage of each pp group (tied embeddings)
    embd_lists = []
    for ranks in ga(("pp",)):
        embd_lists.append(sorted({ranks[0], ranks[-1]}))
    st.embd = _make_groups(embd_lists, rank, backend, timeout=timeout)

    st.virtual_pp_size = virtual_pipeline_model_parallel_size
    st.virtual_pp_rank = 0 if virtual_pipeline_model_parallel_size else None
    st.initialized = True
    return st


# ---- reloadable communicators ------------------------------------------------------------------------------
# In colocated mode the trainer sleeps while the rollout engine owns the GPU. NCCL communicators of a large layout hold
# gigabytes of buffers (the reference measures > 10 GB, docs/en/blogs/release_v0.1.0.md:92), so they are torn down for
# the rollout phase and rebuilt at wake-up. Because every group in this package is fetched through the getters below
# (nothing caches a handle: buffers take a getter, not a group), this needs no patching of torch.distributed as in the
# reference (slime/utils/reloadable_process_group.py:145-270): release destroys WORLD (which shuts down every subgroup in
# one global order, the only order that cannot deadlock pipeline ranks with overlapping subgroups), keeps the rendezvous
# store alive, and leaves a gloo WORLD on a fresh PrefixStore namespace for host-side coordination; reload replaces
# it by a device WORLD on the next namespace and recreates every subgroup from the remembered layout.
def communicators_released() -> bool:
    return getattr(_STATE, "released", False)


def release_communicators() -> bool:
    """Destroy every device communicator of this process. Topology queries (sizes, ranks, rank lists) keep working;
    group getters return None until ``reload_communicators``. Returns False when there was nothing to release."""
    from torch.distributed.distributed_c10d import PrefixStore, _get_default_store

    st = _STATE
    if not (dist.is_available() and dist.is_initialized()) or communicators_released():
        return False
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    info = getattr(st, "world_info", None)
    if info is None:
        info = st.world_info = dict(backend=str(dist.get_backend()), store=_get_default_store(), rank=dist.get_rank(),
                                    world=dist.get_world_size(), generation=0)  # fmt: skip
    dist.barrier()
    dist.destroy_process_group()  # WORLD and, with it, every subgroup
    for a in ParallelState.AXES:
        ax = getattr(st, a)
        ax.group = ax.gloo_group = None
    info["generation"] += 1
    dist.init_process_group("gloo", store=PrefixStore(f"slime-b200-world-{info['generation']}-gloo", info["store"]),
                            rank=info["rank"], world_size=info["world"])  # fmt: skip
    st.released = True
    return True


def reload_communicators() -> bool:
    """Inverse of ``release_communicators``: device WORLD and every subgroup are recreated with the same ranks."""
    from torch.distributed.distributed_c10d import PrefixStore

    st = _STATE
    if not communicators_released():
        return False
    info, layout, vpp_rank = st.world_info, dict(st.layout_args), st.virtual_pp_rank
    dist.barrier()  # still the temporary gloo WORLD: no device communicator is created before every rank is here
    dist.destroy_process_group()
    info["generation"] += 1
    kw = {"timeout": layout["timeout"]} if layout.get("timeout") is not None else {}
    dist.init_process_group(info["backend"], store=PrefixStore(f"slime-b200-world-{info['generation']}", info["store"]),
                            rank=info["rank"], world_size=info["world"], **kw)  # fmt: skip
    initialize_model_parallel(**layout)
    _STATE.world_info, _STATE.virtual_pp_rank, _STATE.released = info, vpp_rank, False
    return True


def destroy_model_parallel():
    st = _STATE
    if dist.is_available() and dist.is_initialized():
        for a in ParallelState.AXES:
            ax = getattr(st, a)
            for g in (ax.group, ax.gloo_group):
                if g is not None:
                    try:
                        dist.destroy_process_group(g)
                    except Exception:
                        pass
    st.reset()


def model_parallel_is_initialized() -> bool:
    return _STATE.initialized


# ---- Megatron-style query surface (names kept so hook code ports 1:1) -------
def get_tensor_model_parallel_group():
    return _STATE.tp.group


def get_tensor_model_parallel_world_size() -> int:
    return _STATE.tp.size


def get_tensor_model_parallel_rank() -> int:
    return _STATE.tp.rank


def get_tensor_model_parallel_ranks() -> list[int]:
    return _STATE.tp.ranks


def get_tensor_model_parallel_src_rank() -> int:
    return _STATE.tp.ranks[0]


def get_pipeline_model_parallel_group():
    return _STATE.pp.group


def get_pipeline_model_parallel_world_size() -> int:
    return _STATE.pp.size


def get_pipeline_model_parallel_rank() -> int:
    return _STATE.pp.rank


def get_pipeline_model_parallel_ranks() -> list[int]:
    return _STATE.pp.ranks


def get_pipeline_model_parallel_next_rank() -> int:
    r = _STATE.pp
    return r.ranks[(r.rank + 1) % r.size]


def get_pipeline_model_parallel_prev_rank() -> int:
    r = _STATE.pp
    return r.ranks[(r.rank - 1) % r.size]


def is_pipeline_first_stage(ignore_virtual: bool = True) -> bool:
    if not ignore_virtual and _STATE.virtual_pp_size and _STATE.virtual_pp_rank != 0:
        return False
    return _STATE.pp.rank == 0


def is_pipeline_last_stage(ignore_virtual: bool = True) -> bool:
    if not ignore_virtual and _STATE.virtual_pp_size and _STATE.virtual_pp_rank != _STATE.virtual_pp_size - 1:
        return False
    return _STATE.pp.rank == _STATE.pp.size - 1


def get_virtual_pipeline_model_parallel_world_size():
    return _STATE.virtual_pp_size


def get_virtual_pipeline_model_parallel_rank():
    return _STATE.virtual_pp_rank


def set_virtual_pipeline_model_parallel_rank(r):
    _STATE.virtual_pp_rank = r


def get_context_parallel_group():
    return _STATE.cp.group


def get_context_parallel_world_size() -> int:
    return _STATE.cp.size


def get_context_parallel_rank() -> int:
    return _STATE.cp.rank


def get_context_parallel_global_ranks() -> list[int]:
    return _STATE.cp.ranks


def get_data_parallel_group(with_context_parallel: bool = False):
    return (_STATE.dp_cp if with_context_parallel else _STATE.dp).group


def get_data_parallel_group_gloo(with_context_parallel: bool = False):
    return (_STATE.dp_cp if with_context_parallel else _STATE.dp).gloo_group


def get_data_parallel_world_size(with_context_parallel: bool = False) -> int:
    return (_STATE.dp_cp if with_context_parallel else _STATE.dp).size


def get_data_parallel_rank(with_context_parallel: bool = False) -> int:
    return (_STATE.dp_cp if with_context_parallel else _STATE.dp).rank


def get_data_parallel_ranks(with_context_parallel: bool = False) -> list[int]:
    return (_STATE.dp_cp if with_context_parallel else _STATE.dp).ranks


def get_expert_model_parallel_group():
    return _STATE.ep.group


def get_expert_model_parallel_world_size() -> int:
    return _STATE.ep.size


def get_expert_model_parallel_rank() -> int:
    return _STATE.ep.rank


def get_expert_model_parallel_ranks() -> list[int]:
    return _STATE.ep.ranks


def get_expert_tensor_parallel_group():
    return _STATE.etp.group


def get_expert_tensor_parallel_world_size() -> int:
    return _STATE.etp.size


def get_expert_tensor_parallel_rank() -> int:
    return _STATE.etp.rank


def get_expert_data_parallel_group():
    return _STATE.edp.group


def get_expert_data_parallel_world_size() -> int:
    return _STATE.edp.size


def get_expert_data_parallel_rank() -> int:
    return _STATE.edp.rank


def get_model_parallel_group():
    return _STATE.mp.group


def get_embedding_group():
    return _STATE.embd.group


def get_tensor_and_context_parallel_group():
    return _STATE.tp_cp.group


def is_main_rank() -> bool:
    """The rank that logs: tp 0, dp(+cp) 0, last pipeline stage (where the loss lives)."""
    return _STATE.tp.rank == 0 and _STATE.dp_cp.rank == 0 and is_pipeline_last_stage()


def set_cp_for_testing(size: int, rank: int, group=None):
    """Pin the CP coordinates without building groups (multi-process CPU tests)."""
    _STATE.cp = _Axis(size=size, rank=rank, group=group, ranks=list(range(size)))
    _STATE.initialized = True


def set_axis_for_testing(name: str, size: int, rank: int, group=None, ranks=None):
    setattr(_STATE, name, _Axis(size=size, rank=rank, group=group, ranks=ranks or list(range(size))))
    _STATE.initialized = True


def all_reduce_scalar(value: float, op=None, group=None) -> float:
    if not (dist.is_available() and dist.is_initialized()):
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu")
    dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=group)
    return float(t.item())
