"""Process topology: a (pp, dp, tp) grid of ranks and its process groups.

Rank order is pipeline-major, tensor-minor: ``rank = (pp_idx * dp + dp_idx) *
tp + tp_idx``, so the ranks of one tensor-parallel group are adjacent GPUs.
On an NVSwitch box every pair of GPUs is equidistant, hence no placement
trade-off between the axes; tensor-minor just keeps the chattiest group on
consecutive device ids.

The object answers the three questions schedules and ``build`` ask of a
topology - "which ranks form the groups along axis X"
(``get_axis_comm_lists``), "which ranks have coordinate c on axis X"
(``filter_match``) and "how long is axis X" (``get_dim``) - and creates the
``torch.distributed`` groups.  Axis aliases: ``pipe``=pp, ``data``=dp,
``model``=tp.

Parity: replaces the DeepSpeed ``PipeModelDataParallelTopology`` used by the
reference (examples/utils.py:57-74, slapo/build.py:73-99).
"""
from __future__ import annotations

import itertools

import torch.distributed as dist

_ALIASES = {"pipe": "pp", "pipeline": "pp", "data": "dp", "model": "tp", "tensor": "tp"}
_AXES = ("pp", "dp", "tp")


class DeviceMesh:
    def __init__(self, pp: int = 1, dp: int = 1, tp: int = 1, rank: int | None = None,
                 create_groups: bool = True):
        self.dims = {"pp": pp, "dp": dp, "tp": tp}
        self.world_size = pp * dp * tp
        if rank is None:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        self.rank = rank
        self.groups = {axis: None for axis in _AXES}
        # (lower stage, "fwd" | "bwd") -> 2-rank group of this rank's pipeline link in that
        # direction (only the links this rank is an end of)
        self.p2p_groups = {}
        if create_groups and dist.is_available() and dist.is_initialized():
            if dist.get_world_size() != self.world_size:
                raise ValueError(f"mesh {self.dims} needs {self.world_size} ranks, "
                                 f"world has {dist.get_world_size()}")
            self._create_groups()

    # ---- coordinates ------------------------------------------------- #
    @staticmethod
    def _axis(name):
        name = _ALIASES.get(name, name)
        if name not in _AXES:
            raise ValueError(f"unknown axis {name}")
        return name

    def get_dim(self, axis) -> int:
        return self.dims[self._axis(axis)]

    def get_rank(self, **coords) -> int:
        c = {self._axis(k): v for k, v in coords.items()}
        return (c.get("pp", 0) * self.dims["dp"] + c.get("dp", 0)) * self.dims["tp"] + c.get("tp", 0)

    def get_coord(self, rank=None) -> dict:
        rank = self.rank if rank is None else rank
        tp = rank % self.dims["tp"]
        dp = (rank // self.dims["tp"]) % self.dims["dp"]
        pp = rank // (self.dims["tp"] * self.dims["dp"])
        return {"pp": pp, "dp": dp, "tp": tp}

    def filter_match(self, **coords) -> list[int]:
        want = {self._axis(k): v for k, v in coords.items()}
        return [r for r in range(self.world_size)
                if all(self.get_coord(r)[a] == v for a, v in want.items())]

    def get_axis_comm_lists(self, axis) -> list[list[int]]:
        axis = self._axis(axis)
        others = [a for a in _AXES if a != axis]
        lists = []
        for combo in itertools.product(*(range(self.dims[a]) for a in others)):
            fixed = dict(zip(others, combo))
            lists.append([self.get_rank(**fixed, **{axis: i}) for i in range(self.dims[axis])])
        return lists

    # ---- groups ------------------------------------------------------ #
    def _create_groups(self):
        for axis in _AXES:
            for ranks in self.get_axis_comm_lists(axis):
                # every rank must take part in every new_group call
                group = dist.new_group(ranks) if len(ranks) > 1 else None
                if self.rank in ranks:
                    self.groups[axis] = group
        # Pipeline links: one 2-rank group per adjacent stage pair AND direction, so that every
        # direction has its own communicator (on GPUs: its own NCCL stream).  Activations going
        # down the pipeline and gradients coming back never queue behind each other, both ends
        # of a communicator issue its transfers in micro-batch order, and plain (unbatched)
        # isend / irecv cannot dead-lock.
        for stage in range(self.dims["pp"] - 1):
            for dp in range(self.dims["dp"]):
                for tp in range(self.dims["tp"]):
                    pair = [self.get_rank(pp=stage, dp=dp, tp=tp),
                            self.get_rank(pp=stage + 1, dp=dp, tp=tp)]
                    for direction in ("fwd", "bwd"):
                        group = dist.new_group(pair)
                        if self.rank in pair:
                            self.p2p_groups[(stage, direction)] = group

    @property
    def schedule_group(self):
        """What to pass as ``group=`` to ``create_schedule`` / ``apply_schedule``: the
        tensor-parallel group, or ``False`` - "no tensor parallelism" - when ``tp == 1``
        (``None`` would mean the whole job, i.e. sharding over data / pipeline peers)."""
        return self.groups["tp"] if self.dims["tp"] > 1 else False

    tp_group = property(lambda self: self.groups["tp"])
    dp_group = property(lambda self: self.groups["dp"])
    pp_group = property(lambda self: self.groups["pp"])
    tp_rank = property(lambda self: self.get_coord()["tp"])
    dp_rank = property(lambda self: self.get_coord()["dp"])
    pp_rank = property(lambda self: self.get_coord()["pp"])
    tp_size = property(lambda self: self.dims["tp"])
    dp_size = property(lambda self: self.dims["dp"])
    pp_size = property(lambda self: self.dims["pp"])

    def stage_ranks(self, stage: int) -> list[int]:
        return self.filter_match(pp=stage)

    def prev_stage_rank(self):
        c = self.get_coord()
        return None if c["pp"] == 0 else self.get_rank(pp=c["pp"] - 1, dp=c["dp"], tp=c["tp"])

    def next_stage_rank(self):
        c = self.get_coord()
        if c["pp"] == self.dims["pp"] - 1:
            return None
        return self.get_rank(pp=c["pp"] + 1, dp=c["dp"], tp=c["tp"])

    def __repr__(self):
        d = self.dims
        return f"DeviceMesh(pp={d['pp']}, dp={d['dp']}, tp={d['tp']}, rank={self.rank})"


def generate_pipeline_cuts(num_layers: int, num_pp: int, is_encoder_decoder: bool = False):
    """Indices of the layers after which an even pipeline split cuts:
    ``generate_pipeline_cuts(24, 4) -> [5, 11, 17]``.  For encoder-decoder
    models returns one list per half (``num_pp`` must be even)."""
    if is_encoder_decoder:
        if num_pp % 2 != 0:
            raise ValueError("encoder-decoder models need an even number of stages")
        half = num_pp // 2
        return [generate_pipeline_cuts(num_layers, half), generate_pipeline_cuts(num_layers, half)]
    per_stage = num_layers // num_pp
    return [per_stage * i - 1 for i in range(1, num_pp)]
