"""Steps as captured CUDA graphs: decode steps, and steps that bring prompts.

A decode step is a few hundred small kernels; launched one by one their launch cost exceeds
their run time. So the step for a given number of rows (rounded up to a bucket, the rest
padding) and a given bound on the positions is captured once and replayed. The graph reads
its step from a StepBatch whose device buffers never move; each replay is preceded by one
small host-to-device copy of that step's indices (or, with `advance`, by a kernel that moves
every row one position on, so that a loop can run without the host).

A graph holds addresses: of the workspace, the cache, the rotary tables. If the workspace has
grown since the capture (its generation changed), the graph is captured again.

A step that brings prompts is a few hundred launches too, each costing the host some ten
microseconds: for a small model that is as long as the GPU works on them. Such steps are captured per
(rows, sequences, wanted rows), each rounded up to a bucket, the second time a shape comes by (a
shape seen once is not worth a capture); the step's work lists for the attention kernels travel in
the StepBatch like its other indices, so a replay needs nothing from the host but that one copy. Whether a
model's steps may be captured at all is the engine's question to the model's parts (engine.capturable).
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
    def __init__(self, engine, rows, position_bound, seqs=None, logit_rows=None):
        self.engine, self.rows, self.position_bound = engine, rows, position_bound
        device = engine.model.ctx.device
        self.batch = StepBatch(rows, rows if seqs is None else seqs, rows if logit_rows is None else logit_rows, device,
                               plans=engine.model.step_plans())
        self.batch.position_bound = position_bound
        self.graph = None
        self.generation = -1
        self.logits = None

    def capture(self, sequences):
        model = self.engine.model
        self.batch.fill(sequences, pad_logits=True)
        # once outside a capture: loads the kernel libraries, sets function attributes, sizes the workspace
        side = torch.cuda.Stream(device=model.ctx.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.engine.forward(self.batch)
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
                self.logits = self.engine.forward(self.batch)
        finally:
            if collecting:
                gc.enable()
        self.n_kernels = ops.LAUNCHES - before  # kernels one replay runs
        self.generation = model.ws.generation

    def run(self, sequences, tokens_dev=None):
        """Replay for this step's sequences; returns the logits of its wanted rows (for a decode step: of
        the first len(sequences) rows). tokens_dev (int32 on the device, one per sequence): the step's tokens,
        instead of the sequences' own (which the host may not know yet)."""
        if self.graph is None or self.generation != self.engine.model.ws.generation:
            self.capture(sequences)
        self.batch.fill(sequences, pad_logits=True)
        if tokens_dev is not None:
            self.batch.tokens[:len(sequences)].copy_(tokens_dev[:len(sequences)])
        self.graph.replay()
        return self.logits[:sum(len(s.want) for s in sequences)]

    def replay_advanced(self):
        """Replay after moving every row one position on, on the device; the tokens are whatever the
        token buffer holds (a sampler may have written them there). Nothing comes from the host."""
        if self.position_bound is not None and self.batch.max_len_after + 1 > self.position_bound:
            raise ValueError(f"a row would move to position {self.batch.max_len_after}, beyond the bound "
                             f"{self.position_bound} this graph was captured for")
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


def prompt_bucket(n):
    """Rows of a captured prompt step: powers of two up to 128, then steps of an eighth to a sixteenth of the size."""
    if n <= 128:
        return max(16, 1 << (n - 1).bit_length())
    step = max(128, 1 << (n.bit_length() - 4))
    return -(-n // step) * step


class PromptGraphs:
    """Captured steps that bring several tokens of some sequence. A shape is captured when it comes by a
    second time; at most `keep` graphs are kept (the least recently used goes)."""

    def __init__(self, engine, keep=16):
        self.engine, self.keep = engine, keep
        self.graphs, self.seen = {}, {}
        self.captured = self.replayed = 0

    def key(self, sequences):
        rows = sum(len(s.tokens) for s in sequences)
        wanted = sum(len(s.want) for s in sequences)
        return (prompt_bucket(rows), 1 << (len(sequences) - 1).bit_length(), 1 << max(0, wanted - 1).bit_length())

    def takes(self, sequences):
        """Whether this step is replayed (or captured now). Steps of one token per sequence are the decode
        graphs' (or run as they are)."""
        if all(len(s.tokens) == 1 for s in sequences):
            return False
        key = self.key(sequences)
        if key in self.graphs:
            return True
        self.seen[key] = self.seen.get(key, 0) + 1
        if len(self.seen) > 4096:
            self.seen.clear()
        return self.seen[key] >= 2

    def run(self, sequences):
        key = self.key(sequences)
        graph = self.graphs.pop(key, None)
        if graph is None:
            if len(self.graphs) >= self.keep:
                self.graphs.pop(next(iter(self.graphs)))
            graph = DecodeGraph(self.engine, key[0], None, seqs=key[1], logit_rows=key[2])
        self.graphs[key] = graph  # most recently used last
        fresh = graph.graph is None or graph.generation != self.engine.model.ws.generation
        logits = graph.run(sequences)
        self.captured += fresh
        self.replayed += 1
        return logits, graph.batch
