"""bin/trace_run against the plain implementation: every way of cutting and batching the same
requests must give the same logits, in float32 and in bfloat16, for three tiny configurations.

One trace_run process per (configuration, dtype) replays, one after another:
  1. each request alone and whole (logits at every position),
  2. each request alone with its last 32 tokens one by one (tools/check.py:70-75, --chunk 1),
  3. batches of unequal lengths that start together, whose shorter requests end earlier, one batch
     after another in a cache just large enough for one batch, so slots and pages are used again,
  4. a long decode, token by token, across many pages (and many turns of a windowed ring),
  5. the first tokens of a sequence: prompts of one, two and three tokens.
"""
import numpy as np
import pytest

from helpers import TINY, TraceRun, assert_logits, make_model_folder, random_tokens
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

# lengths around the page size of 64 and its multiples on purpose
LENGTHS = [37, 70, 5, 129, 64, 33, 128, 65]


def ceil64(n):
    return -(-n // 64) * 64


class Case:
    """Requests of a configuration and their logits by the plain implementation (made once per dtype)."""
    _made = {}

    def __init__(self, folder, name, dtype):
        self.cfg, self.w = plain.load(folder)
        self.vocab = self.cfg["vocab"]
        rng = np.random.default_rng(100 + ord(name[0]))
        self.requests = {f"r{i}": random_tokens(rng, n, self.vocab) for i, n in enumerate(LENGTHS)}
        long_n = min(330, TINY[name]["cfg"]["max_position_embeddings"] - 8)
        self.requests["long"] = random_tokens(rng, long_n, self.vocab)
        for i in (1, 2, 3):
            self.requests[f"first{i}"] = random_tokens(rng, i, self.vocab)
        self.rnd = plain.bf16_round if dtype == "bfloat16" else None
        self.dtype = dtype
        self._want, self._noise, self.whole = {}, {}, {}

    def want(self, rid):
        if rid not in self._want:
            self._want[rid] = plain.forward(self.cfg, self.w, self.requests[rid], rnd=self.rnd)
        return self._want[rid]

    def noise(self, rid):
        """The rounding noise of this dtype on this request (see helpers.assert_logits)."""
        if rid not in self._noise:
            exact = plain.forward(self.cfg, self.w, self.requests[rid])
            if self.dtype == "bfloat16":
                self._noise[rid] = float(np.abs(self.want(rid) - exact).max())
            else:
                self._noise[rid] = float(np.abs(exact - plain.forward64(self.cfg, self.w, self.requests[rid])).max())
        return self._noise[rid]

    def check(self, got, rid, rows, what):
        assert_logits(got, self.want(rid)[rows], self.dtype, f"{what} of {rid}", noise=self.noise(rid))
        # In float32 every reduction's order depends on the element's own place alone, so however the work is cut
        # and whatever else is in the batch, a position's logits are the same bits (abacus's own whole-sequence,
        # five-token and one-by-one runs are bit-identical too; tools/check.py:70-75 runs both cuts for this).
        if self.dtype == "float32":
            if rid not in self.whole:
                assert rows == slice(0, len(self.requests[rid])), "the whole request comes first"
                self.whole[rid] = np.array(got)
            else:
                assert np.array_equal(got, self.whole[rid][rows]), f"{what} of {rid}: not the bits of the whole request"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: make_model_folder(root, name) for name in TINY}


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16"),
                                         ("C", "float32"), ("C2", "bfloat16"), ("D", "float32"), ("D", "bfloat16")])
def test_replay(folders, tmp_path, name, dtype):
    case = Case(folders[name], name, dtype)
    R, V = case.requests, case.vocab
    batches = [["r0", "r1", "r2"], ["r3", "r4", "r5", "r6"], ["r7", "r2", "r0", "r1"]]
    max_tokens = max(max(sum(ceil64(len(R[r])) for r in b) for b in batches), ceil64(len(R["long"])))
    run = TraceRun(folders[name], dtype, tmp_path / "out", max_tokens)
    try:
        # 1. alone and whole
        for rid in [f"r{i}" for i in range(len(LENGTHS))]:
            n = len(R[rid])
            got = run.step([(rid, R[rid], list(range(n)))], end=[rid])
            case.check(got.reshape(n, V), rid, slice(0, n), f"{name} whole")
        # 2. last 32 one by one
        for rid in [f"r{i}" for i in range(len(LENGTHS))]:
            toks, n = R[rid], len(R[rid])
            head = max(n - 32, 0)
            rows = []
            if head:
                rows.append(run.step([(rid, toks[:head], [head - 1])]).reshape(1, V))
            for i in range(head, n):
                rows.append(run.step([(rid, [toks[i]], [0])], end=[rid] if i == n - 1 else []).reshape(1, V))
            first = head - 1 if head else 0
            case.check(np.concatenate(rows), rid, slice(first, n), f"{name} last 32 one by one")
        # 3. unequal batches, shorter requests end earlier, batch after batch
        for b in batches:
            split = {rid: max(1, len(R[rid]) - (7 + 5 * i)) for i, rid in enumerate(b)}  # prompt | decoded part
            got = run.step([(rid, R[rid][:split[rid]], list(range(split[rid]))) for rid in b],
                           end=[rid for rid in b if split[rid] == len(R[rid])])
            at = 0
            for rid in b:
                case.check(got[at * V:(at + split[rid]) * V].reshape(split[rid], V), rid, slice(0, split[rid]),
                           f"{name} batch {b} prompt")
                at += split[rid]
            live = [rid for rid in b if split[rid] < len(R[rid])]
            k = 0
            while live:
                ends = [rid for rid in live if split[rid] + k == len(R[rid]) - 1]
                got = run.step([(rid, [R[rid][split[rid] + k]], [0]) for rid in live], end=ends)
                for j, rid in enumerate(live):
                    case.check(got[j * V:(j + 1) * V].reshape(1, V), rid, slice(split[rid] + k, split[rid] + k + 1),
                               f"{name} batch {b} decode {k}")
                live = [rid for rid in live if rid not in ends]
                k += 1
        # 4. long decode, one token at a time after a 40-token prompt (whole first, for the comparison of cuts)
        toks, n = R["long"], len(R["long"])
        for rid in ["long", "first1", "first2", "first3"]:
            m = len(R[rid])
            case.check(run.step([(rid, R[rid], list(range(m)))], end=[rid]).reshape(m, V), rid, slice(0, m), f"{name} whole")
        rows = [run.step([("long", toks[:40], [39])]).reshape(1, V)]
        for i in range(40, n):
            rows.append(run.step([("long", [toks[i]], [0])], end=["long"] if i == n - 1 else []).reshape(1, V))
        case.check(np.concatenate(rows), "long", slice(39, n), f"{name} long decode")
        # 5. the first tokens of a sequence, as one batch of very short prompts and then decoded
        ids = ["first1", "first2", "first3"]
        got = run.step([(rid, R[rid][:1], [0]) for rid in ids], end=["first1"])
        for j, rid in enumerate(ids):
            case.check(got[j * V:(j + 1) * V].reshape(1, V), rid, slice(0, 1), f"{name} first token")
        got = run.step([(rid, R[rid][1:2], [0]) for rid in ids[1:]], end=["first2"])
        for j, rid in enumerate(ids[1:]):
            case.check(got[j * V:(j + 1) * V].reshape(1, V), rid, slice(1, 2), f"{name} second token")
        got = run.step([("first3", R["first3"][2:3], [0])], end=["first3"])
        case.check(got.reshape(1, V), "first3", slice(2, 3), f"{name} third token")
        # a step that wants nothing writes nothing
        assert run.step([("quiet", R["r2"], [])], end=["quiet"]) is None
    finally:
        run.close()
