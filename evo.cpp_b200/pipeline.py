"""Layer pipeline with one stage per process (torchrun: one rank per GPU).

Rank r holds stage r of the contiguous split of the blocks
(``evo_b200_model_load_slice``: upstream's byte-balanced split up to four
stages, equal block counts beyond).  A prompt moves through the stages as a chunk
wavefront: rank r receives the hidden rows of window j from rank r-1, runs its
blocks over them, and sends them on while rank r-1 already works on window
j+1.  That is legal because every mixer is causal and carries its state from
window to window.  The hand-off is ``torch.distributed`` point-to-point
(NCCL over NVLink on GPUs; gloo in the CPU tests of this schedule): receives
are ordered on the stage's compute stream, sends are asynchronous so a stage
never waits for its successor unless it is about to overwrite rows still in
flight.

Upstream runs the same stage plan inside one process and hands the whole
sequence from device to device (src/cuda/model.cu:2148-2366); the wavefront is
this implementation's addition.
"""
from __future__ import annotations

from typing import Protocol


def window_plan(rows: int, stages: int, chunk: int = 0) -> list[tuple[int, int]]:
    """[(begin, count)] windows of one prompt, each a power of two in [512, 2048]
    rows so that they divide the activation capacity (prompts longer than it
    wrap around): about two windows per stage up to four stages, one per stage
    beyond.  More windows fill the pipeline better, but a 512-row window runs
    the 4096-wide projections at well under half the tensor rate they reach at
    1,024 rows (128 x 128 tiles re-read their operands from L2 twice as often),
    which costs an eight-stage pipeline more than the shorter fill gains."""
    if rows <= 0 or stages <= 0:
        raise ValueError("rows and stages must be positive")
    if chunk <= 0:
        per_stage = 2 if stages <= 4 else 1
        chunk = 512
        while chunk < 2048 and chunk * per_stage * stages < rows:
            chunk *= 2
    return [(begin, min(chunk, rows - begin)) for begin in range(0, rows, chunk)]


class Stage(Protocol):
    """What the schedule needs from the local stage (all calls enqueue work)."""

    def embed(self, begin: int, count: int) -> None: ...   # first stage: tokens -> hidden rows
    def run(self, begin: int, count: int) -> None: ...     # this stage's blocks over hidden rows
    def head(self, begin: int, count: int) -> None: ...    # last stage: final norm + logits of the window


class StagePipeline:
    """Drives one rank's part of the wavefront.

    ``hidden`` is a [capacity, width] tensor aliasing the stage's hidden-row
    buffer; the window at sequence position p is sent from and received into
    rows p % capacity .. directly (prompts longer than the capacity wrap).
    """

    def __init__(self, stage: Stage, hidden, rank: int, world: int, group=None, chunk: int = 0):
        if not 0 <= rank < world:
            raise ValueError("rank outside the pipeline")
        self.stage, self.hidden, self.rank, self.world = stage, hidden, rank, world
        self.group, self.chunk = group, chunk
        self.in_flight: dict[int, object] = {}   # window begin -> pending send of those rows
        self.last_rows = None

    def step(self, rows: int) -> None:
        """One prompt of `rows` tokens through this rank's stage."""
        import torch.distributed as dist

        capacity = self.hidden.shape[0]
        plan = window_plan(rows, self.world, self.chunk)
        if rows > capacity and any(capacity % count for _, count in plan[:-1]):
            raise ValueError("windows of a prompt longer than the hidden-row capacity must divide it")
        if rows != self.last_rows:
            self.drain()       # a different window layout: nothing may still be in flight
            self.last_rows = rows
        for begin, count in plan:
            row = begin % capacity
            pending = self.in_flight.pop(row, None)
            if pending is not None:
                pending.wait()  # these rows are about to be overwritten
            window = self.hidden[row:row + count]
            if self.rank == 0:
                self.stage.embed(begin, count)
            else:
                dist.recv(window, src=self._peer(self.rank - 1), group=self.group)
            self.stage.run(begin, count)
            if self.rank + 1 < self.world:
                self.in_flight[row] = dist.isend(window, dst=self._peer(self.rank + 1), group=self.group)
            else:
                self.stage.head(begin, count)

    def drain(self) -> None:
        for pending in self.in_flight.values():
            pending.wait()
        self.in_flight.clear()

    def _peer(self, pipeline_rank: int) -> int:
        import torch.distributed as dist

        if self.group is None:
            return pipeline_rank
        return dist.get_global_rank(self.group, pipeline_rank)


class DeviceRows:
    """CUDA-array-interface view of a BF16 [rows, width] device buffer owned by
    the runtime library, so torch can alias it without a copy."""

    def __init__(self, address: int, rows: int, width: int):
        self.__cuda_array_interface__ = {"shape": (rows, width), "typestr": "<i2", "data": (address, False),
                                         "version": 2, "strides": None}


def alias_hidden_rows(context, rows: int, width: int, device):
    """torch BF16 [rows, width] tensor over the context's hidden-row buffer."""
    import torch

    raw = torch.as_tensor(DeviceRows(context.slice_hidden(), rows, width), device=device)
    return raw.view(torch.bfloat16)


class ContextStage:
    """`Stage` over a sliced runtime context; `tokens` is a device int32/uint32
    tensor holding the prompt (used by the first stage only)."""

    def __init__(self, context, tokens=None):
        self.context, self.tokens = context, tokens
        self.logits_address = None

    def embed(self, begin: int, count: int) -> None:
        self.context.slice_embed(self.tokens.data_ptr() + 4 * begin, begin, count)

    def run(self, begin: int, count: int) -> None:
        self.context.slice_run(begin, count)

    def head(self, begin: int, count: int) -> None:
        self.logits_address = self.context.slice_head(begin, count)
