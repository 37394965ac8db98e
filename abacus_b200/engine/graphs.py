"""Decode steps as captured CUDA graphs.

A decode step is a few hundred small kernels; launched one by one their launch cost exceeds
their run time. So the step for a given number of rows (rounded up to a bucket, the rest
padding) and a given bound on the positions is captured once and replayed. The graph reads
its step from a StepBatch whose device buffers never move; each replay is preceded by one
small host-to-device copy of that step's indices (or, with `advance`, by a kernel that moves
every row one position on, so that a loop can run without the host).

A graph holds addresses: of the workspace, the cache, the rotary tables. If the workspace has
grown since the capture (its generation changed), the graph is captured again.
"""
import gc

import torch

from .batch import StepBatch

ROW_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
POSITION_STEP = 1024


def row_bucket(n):
    for b in ROW_BUCKETS:
        if n <= b:
            return b
    return None


class DecodeGraph:
    def __init__(self, engine, rows, position_bound):
        self.engine, self.rows, self.position_bound = engine, rows, position_bound
        device = engine.model.ctx.device
        self.batch = StepBatch(rows, rows, rows, device)
        self.batch.position_bound = position_bound
        self.graph = None
        self.generation = -1
        self.logits = None

    def capture(self, sequences):
        model, cache = self.engine.model, self.engine.cache
        self.batch.fill(sequences, pad_logits=True)
        # once outside a capture: loads the kernel libraries, sets function attributes, sizes the workspace
        side = torch.cuda.Stream(device=model.ctx.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            model.forward(self.batch, cache)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..kernels import ops
        before = ops.LAUNCHES
        self.graph = torch.cuda.CUDAGraph()
        # Python's collector must not run inside the capture: if it frees an earlier engine's graphs or
        # buffers there, the memory calls it makes invalidate the capture in progress.
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = model.forward(self.batch, cache)
        finally:
            if collecting:
                gc.enable()
        self.n_kernels = ops.LAUNCHES - before  # kernels one replay runs
        self.generation = model.ws.generation

    def run(self, sequences):
        """Replay for this step's sequences (each with one token, logits wanted); returns the logits
        of the first len(sequences) rows."""
        if self.graph is None or self.generation != self.engine.model.ws.generation:
            self.capture(sequences)
        self.batch.fill(sequences, pad_logits=True)
        self.graph.replay()
        return self.logits[:len(sequences)]

    def replay_advanced(self):
        """Replay after moving every row one position on, on the device; the tokens are whatever the
        token buffer holds (a sampler may have written them there). Nothing comes from the host."""
        self.batch.advance_on_device()
        self.graph.replay()
        return self.logits[:self.batch.n_seqs]


class DecodeGraphs:
    def __init__(self, engine):
        self.engine, self.graphs = engine, {}

    def takes(self, sequences):
        return (row_bucket(len(sequences)) is not None
                and all(len(s.tokens) == 1 and list(s.want) == [0] for s in sequences))

    def get(self, sequences):
        rows = row_bucket(len(sequences))
        top = max(s.start + 1 for s in sequences)
        bound = min(-(-top // POSITION_STEP) * POSITION_STEP, max(self.engine.max_context, top))
        key = (rows, bound)
        if key not in self.graphs:
            self.graphs[key] = DecodeGraph(self.engine, rows, bound)
        return self.graphs[key]

    def run(self, sequences):
        return self.get(sequences).run(sequences)
