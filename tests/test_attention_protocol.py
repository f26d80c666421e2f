"""The attention kernels' synchronisation protocols, model-checked on the CPU.

`fb_attention_forward` (flint_b200/csrc/attention.cu) hands work between a TMA producer, an
MMA-issuing warp and sixteen softmax warps through mbarriers whose waits carry only a phase
parity. A parity wait is right only while at most one phase of that barrier is outstanding,
and whether that holds depends on how long loads and MMAs take: a wait that is two phases
behind passes early without any error (this happened: the kernel's last wait for P V,
with a cold L2). Timing-dependent mistakes of that kind do not show in a GPU test that happens
to run with warm caches, so this file restates the kernel's barrier protocol (the same
cursors, ring order, buffer rotation and parities) as cooperating generators, runs it under
hundreds of random schedules with random load and MMA latencies, and checks every access
against the data it must see:

* a wait that passes although the phase it was meant for has not completed ("aliased wait");
* S(n + 3) executing before P V(n) has read the buffer, P V(n) before all eight warps wrote P;
* a softmax warp reading scores that are not there yet or already overwritten, rescaling or
  reading O before the P V it needs has finished;
* a ring slot or a query buffer reloaded before its readers are done; a deadlock.

Two tests put two earlier forms of the forward kernel's final waits into the model and require
the checker to find their faults, which is what pins the model's power to find that class of bug.
The second half models the dK/dV kernel (and, with queries and keys exchanged, dQ) the same way.
"""

import random

import pytest

SLOTS = 8          # kFwdSlots
WARPS = 8          # softmax warps per query tile


class Violation(AssertionError):
    pass


def need(condition, message):
    if not condition:
        raise Violation(message)


class Barrier:
    def __init__(self, name, count):
        self.name, self.count, self.arrived, self.completed = name, count, 0, 0

    def arrive(self):
        self.arrived += 1
        if self.arrived == self.count:
            self.arrived = 0
            self.completed += 1

    def passed(self, parity):
        return (self.completed & 1) != parity


class Cursor:
    """FwdCursor with enter()/advance(): item `round` of this CTA, key tile j, query tile t."""

    def __init__(self, items, round_=0):
        self.items, self.round, self.j, self.t = items, round_, 0, 0

    @property
    def valid(self):
        return self.round < len(self.items)

    @property
    def qb(self):
        return self.items[self.round]

    def advance(self):
        self.t ^= 1
        if self.t == 0:
            self.j += 1
            if self.j > self.qb:
                self.round, self.j = self.round + 1, 0

    def key(self):
        return (self.round, self.j, self.t)


class Model:
    def __init__(self, items, seed, variant="kernel"):
        self.items = items                      # query tile index (qb) of each item
        self.rng = random.Random(seed)
        # "kernel": what the kernel does. Two earlier forms, kept to show that the checker finds
        # their faults: "single" waits only for the last P V; "after_arrival" waits for the last
        # but one as well, but after the warp's last arrival.
        self.variant = variant
        self.bar = {}
        for b in range(2):
            self.bar["q_full", b] = Barrier(f"q_full{b}", 1)
            self.bar["q_empty", b] = Barrier(f"q_empty{b}", 1)
            self.bar["pv_done", b] = Barrier(f"pv_done{b}", 1)
        for b in range(3):
            self.bar["s_full", b] = Barrier(f"s_full{b}", 1)
            self.bar["p_ready", b] = Barrier(f"p_ready{b}", WARPS)
        for s in range(SLOTS):
            self.bar["slot_full", s] = Barrier(f"slot_full{s}", 1)
            self.bar["slot_empty", s] = Barrier(f"slot_empty{s}", 1)
        self.pair_sync = {}                     # (tile, quadrant, count) -> arrivals
        # Data state.
        self.slot_content = [None] * SLOTS      # tile id now readable in the slot
        self.slot_readers_done = [True] * SLOTS
        self.q_content = [None, None]           # round whose query tiles the buffer holds
        self.q_reads_pending = [0, 0]
        self.s_started, self.s_done, self.pv_started, self.pv_done = set(), set(), set(), set()
        self.p_written = {}                     # step -> warps that wrote their probabilities
        self.tma = []                           # pending loads: (kind, payload)
        self.pipe = []                          # MMA groups and commits, in issue order
        self.steps = []                         # step number -> (round, j, t)
        c = Cursor(items)
        while c.valid:
            self.steps.append(c.key())
            c.advance()
        self.step_of = {key: n for n, key in enumerate(self.steps)}

    # ---- waits -----------------------------------------------------------------------------
    def wait(self, kind, index, parity, phase):
        """Generator: blocks until the barrier passes for `parity`; `phase` is the phase index the
        kernel means, which must then really be complete."""
        bar = self.bar[kind, index]
        while not bar.passed(parity & 1):
            yield
        need(bar.completed > phase, f"aliased wait on {bar.name}: meant phase {phase}, "
                                    f"{bar.completed} completed")

    # ---- roles -----------------------------------------------------------------------------
    def producer(self):
        slot, phase = 0, 0
        keys, values = Cursor(self.items), Cursor(self.items)
        loads = {"k": 0, "v": 0}
        ahead = 0
        uses = [0] * SLOTS

        def load(kind, cursor):
            nonlocal slot, phase
            yield from self.wait("slot_empty", slot, phase ^ 1, uses[slot] - 1)
            need(self.slot_readers_done[slot], f"slot {slot} reloaded while its tile is still read")
            self.slot_content[slot] = None
            self.tma.append(("tile", (slot, (kind,) + cursor.key())))
            uses[slot] += 1
            loads[kind] += 1
            slot += 1
            if slot == SLOTS:
                slot, phase = 0, phase ^ 1

        while values.valid:
            if ahead >= 3:
                yield from load("v", values)
                values.advance()
            if keys.valid:
                if keys.j == 0 and keys.t == 0:
                    b = keys.round & 1
                    if keys.round >= 2:
                        yield from self.wait("q_empty", b, ((keys.round >> 1) - 1) & 1,
                                             (keys.round >> 1) - 1)
                        need(self.q_reads_pending[b] == 0, "query buffer reloaded while still read")
                    self.q_content[b] = None
                    self.tma.append(("q", (b, keys.round)))
                yield from load("k", keys)
                keys.advance()
            ahead += 1
            yield

    def mma_warp(self):
        slot, phase = 0, 0
        uses = [0] * SLOTS
        ahead = Cursor(self.items)
        issued = 0

        def next_tile(expect):
            yield from self.wait("slot_full", slot, phase, uses[slot])
            need(self.slot_content[slot] == expect,
                 f"slot {slot} holds {self.slot_content[slot]}, wanted {expect}")
            self.slot_readers_done[slot] = False

        def step_ring():
            nonlocal slot, phase
            uses[slot] += 1
            slot += 1
            if slot == SLOTS:
                slot, phase = 0, phase ^ 1

        def issue_scores():
            nonlocal issued
            if not ahead.valid:
                return
            b = ahead.round & 1
            if ahead.j == 0 and ahead.t == 0:
                yield from self.wait("q_full", b, (ahead.round >> 1) & 1, ahead.round >> 1)
            yield from next_tile(("k",) + ahead.key())
            self.q_reads_pending[b] += 1
            self.pipe.append(("scores", issued, slot, b, ahead.round))
            self.pipe.append(("commit", ("s_full", issued % 3)))
            self.pipe.append(("commit", ("slot_empty", slot)))
            if ahead.t == 1 and ahead.j == ahead.qb:
                self.pipe.append(("commit", ("q_empty", b)))
            step_ring()
            issued += 1
            ahead.advance()

        for _ in range(3):
            yield from issue_scores()
        at = Cursor(self.items)
        n = 0
        while at.valid:
            yield from self.wait("p_ready", n % 3, (n // 3) & 1, n // 3)
            yield from next_tile(("v",) + at.key())
            self.pipe.append(("weighted", n, slot, at.t))
            self.pipe.append(("commit", ("pv_done", at.t)))
            self.pipe.append(("commit", ("slot_empty", slot)))
            step_ring()
            yield from issue_scores()
            at.advance()
            n += 1
            yield

    def softmax_warp(self, tile, quadrant, half):
        before = 0
        for round_, qb in enumerate(self.items):
            for j in range(qb + 1):
                n = 2 * (before + j) + tile
                need(self.steps[n] == (round_, j, tile), "step numbering out of line")
                yield from self.wait("s_full", n % 3, (n // 3) & 1, n // 3)
                need(n in self.s_done and (n + 3) not in self.s_started,
                     f"scores of step {n} read while absent or overwritten")
                yield
                # The pair's exchange of row maxima (a named barrier of the two warps).
                key = (tile, quadrant, before + j)
                self.pair_sync[key] = self.pair_sync.get(key, 0) + 1
                while self.pair_sync[key] < 2:
                    yield
                moved = j > 0 and random.Random(hash((tuple(self.items), n, quadrant))).random() < 0.4
                if moved:
                    yield from self.wait("pv_done", tile, (before + j - 1) & 1, before + j - 1)
                    need((n - 2) in self.pv_done and n not in self.pv_started,
                         f"O rescaled at step {n} without the previous P V done")
                yield
                need((n + 3) not in self.s_started, f"P of step {n} written over newer scores")
                self.p_written[n] = self.p_written.get(n, 0) + 1
                if self.variant == "kernel" and j == qb and qb > 0:
                    # Before the arrival that lets the item's last P V be issued at all.
                    yield from self.wait("pv_done", tile, (before + qb - 1) & 1, before + qb - 1)
                self.bar["p_ready", n % 3].arrive()
                yield
            if self.variant == "after_arrival" and qb > 0:
                yield from self.wait("pv_done", tile, (before + qb - 1) & 1, before + qb - 1)
            yield from self.wait("pv_done", tile, (before + qb) & 1, before + qb)
            last = 2 * (before + qb) + tile
            need(last in self.pv_done, f"O of item {round_} read before its last P V (step {last})")
            need((last + 2) not in self.pv_started or qb + 1 == 0,
                 "O read after the next item's first P V started")
            before += qb + 1
            yield

    # ---- engines ---------------------------------------------------------------------------
    def run_tma(self):
        kind, payload = self.tma.pop(self.rng.randrange(len(self.tma)))   # any order
        if kind == "tile":
            slot, tile = payload
            self.slot_content[slot] = tile
            self.bar["slot_full", slot].arrive()
        else:
            b, round_ = payload
            self.q_content[b] = round_
            self.bar["q_full", b].arrive()

    def run_pipe(self):
        op = self.pipe.pop(0)                                              # in issue order
        if op[0] == "commit":
            kind, index = op[1]
            self.bar[kind, index].arrive()
            if kind == "slot_empty":
                self.slot_readers_done[index] = True
        elif op[0] == "scores":
            _, n, slot, b, round_ = op
            need(self.q_content[b] == round_, f"scores of step {n} read the wrong query tiles")
            need(n < 3 or (n - 3) in self.pv_done, f"S({n}) overwrites P({n - 3}) before its P V")
            self.s_started.add(n)
            self.s_done.add(n)
            self.q_reads_pending[b] -= 1
        else:
            _, n, slot, tile = op
            need(self.p_written.get(n, 0) == WARPS, f"P V({n}) before all warps wrote P")
            need(n < 2 or (n - 2) in self.pv_done, "P V of a tile out of order")
            self.pv_started.add(n)
            self.pv_done.add(n)

    def run(self):
        roles = {"producer": self.producer(), "mma": self.mma_warp()}
        for tile in range(2):
            for quadrant in range(4):
                for half in range(2):
                    roles[f"softmax{tile}.{quadrant}.{half}"] = self.softmax_warp(tile, quadrant, half)
        schedule(self.rng, roles, [(self.tma, self.run_tma), (self.pipe, self.run_pipe)])
        need(not self.tma and len(self.pv_done) == len(self.steps), "work left over at the end")


def schedule(rng, roles, engines):
    """Runs the role generators to completion in a random interleaving: every round each role
    makes a step with probability one half (so any role can fall far behind the others), and
    each engine (pending loads, the tensor pipe's queue) completes one operation with
    probability 0.35. No engine operation for 20,000 rounds while roles still wait is a deadlock."""
    quiet = 0
    while roles:
        names = list(roles)
        rng.shuffle(names)
        for name in names:
            if rng.random() < 0.5:
                continue
            try:
                next(roles[name])
            except StopIteration:
                del roles[name]
        for queue, run in engines:
            if queue and rng.random() < 0.35:
                run()
                quiet = 0
        quiet += 1
        need(quiet < 20000, f"deadlock: {sorted(roles)} still waiting")


ITEM_LISTS = [[0], [1], [7], [0, 0, 0], [2, 1, 0], [7, 4, 1], [3, 3, 3, 3], [0, 7, 0, 5, 1]]


@pytest.mark.parametrize("items", ITEM_LISTS, ids=[str(i) for i in ITEM_LISTS])
def test_forward_protocol_holds_under_random_schedules(items):
    for seed in range(40):
        Model(items, seed).run()


def test_the_checker_notices_a_missing_wait():
    """Waiting only for the item's last P V: some schedule passes that parity wait a phase
    early and reads O without the last key tiles (the mistake the kernel once had)."""
    found = 0
    for seed in range(200):
        try:
            Model([7, 4, 1], seed, variant="single").run()
        except Violation as violation:
            found += 1
            assert "aliased wait" in str(violation) or "O of item" in str(violation)
    assert found > 0


def test_the_checker_notices_a_wait_that_comes_too_late():
    """Waiting for the last but one P V after the warp's last arrival: a slow warp can find both
    complete, and the parity it waits for never comes (the kernel's bounded wait would give up
    after a second). The kernel waits before the arrival instead."""
    found = 0
    for seed in range(200):
        try:
            Model([7], seed, variant="after_arrival").run()
        except Violation as violation:
            found += 1
            assert "deadlock" in str(violation)
    assert found > 0


# ---- the dK/dV kernel -------------------------------------------------------------------------
#
# fb_attention_dkv: the producer fetches an item's K and V tiles (one shared-memory pair,
# refilled once the compute warps have copied the item before into tensor memory) and streams
# 64-query stages through a ring of four; the MMA warp issues the scores of sub-step h + 1
# before it waits for sub-step h's probabilities (two accumulator pairs), then the gradient
# MMAs; sixteen compute warps turn scores into probabilities in place, install the next item's
# K and V after their last sub-step and write the item's gradients out. fb_attention_dq has the
# same protocol with the roles of queries and keys exchanged.

STAGES = 4         # kBwdStages
COMPUTE = 16       # kBwdComputeWarps


class BackwardModel:
    def __init__(self, items, seed):
        self.items = items                     # sub-steps of each item (even numbers)
        self.rng = random.Random(seed)
        self.bar = {("resident", 0): Barrier("resident", 1), ("done", 0): Barrier("done", 1),
                    ("a_ready", 0): Barrier("a_ready", COMPUTE)}
        for b in range(2):
            self.bar["scores_full", b] = Barrier(f"scores_full{b}", 1)
            self.bar["operands_ready", b] = Barrier(f"operands_ready{b}", COMPUTE)
        for s in range(STAGES):
            self.bar["stage_full", s] = Barrier(f"stage_full{s}", 1)
            self.bar["stage_empty", s] = Barrier(f"stage_empty{s}", 1)
        self.tma, self.pipe = [], []
        self.shared_item = None                # item whose K/V the shared-memory pair holds
        self.installed = {}                    # item -> warps that copied it to tensor memory
        self.stage_content = [None] * STAGES
        self.stage_reads = [0] * STAGES        # MMA groups issued on the stage, not yet executed
        self.scores_done, self.scores_started, self.grads_done = set(), set(), set()
        self.written = {}                      # sub-step count -> warps that wrote probabilities
        self.first_count = [sum(items[:i]) for i in range(len(items))]

    def wait(self, kind, index, parity, phase):
        bar = self.bar[kind, index]
        while not bar.passed(parity & 1):
            yield
        need(bar.completed > phase, f"aliased wait on {bar.name}: meant phase {phase}, "
                                    f"{bar.completed} completed")

    def producer(self):
        stage, phase = 0, 0
        uses = [0] * STAGES
        for round_, steps in enumerate(self.items):
            if round_ > 0:
                yield from self.wait("a_ready", 0, (round_ - 1) & 1, round_ - 1)
                need(self.installed.get(round_ - 1, 0) == COMPUTE,
                     "K/V in shared memory replaced before every warp copied them")
            self.shared_item = None
            self.tma.append(("resident", round_))
            for h in range(steps):
                yield from self.wait("stage_empty", stage, phase ^ 1, uses[stage] - 1)
                need(self.stage_reads[stage] == 0, f"stage {stage} refilled while still read")
                self.stage_content[stage] = None
                self.tma.append(("stage", (stage, self.first_count[round_] + h)))
                uses[stage] += 1
                stage += 1
                if stage == STAGES:
                    stage, phase = 0, phase ^ 1
                yield

    def mma_warp(self):
        before = 0
        for round_, steps in enumerate(self.items):
            yield from self.wait("a_ready", 0, round_ & 1, round_)

            def issue_scores(g):
                count = before + g
                stage = count % STAGES
                yield from self.wait("stage_full", stage, (count // STAGES) & 1, count // STAGES)
                need(self.stage_content[stage] == count, f"stage {stage} holds the wrong sub-step")
                self.stage_reads[stage] += 1
                self.pipe.append(("scores", count, stage, round_))
                self.pipe.append(("commit", ("scores_full", g & 1)))

            yield from issue_scores(0)
            for h in range(steps):
                b = h & 1
                count = before + h
                if h + 1 < steps:
                    yield from issue_scores(h + 1)
                yield from self.wait("operands_ready", b, (count >> 1) & 1, count >> 1)
                stage = count % STAGES
                self.stage_reads[stage] += 1
                self.pipe.append(("grads", count, stage))
                self.pipe.append(("commit", ("stage_empty", stage)))
                if h + 1 == steps:
                    self.pipe.append(("commit", ("done", 0)))
                yield
            before += steps

    def compute_warp(self, index):
        def install(round_):
            yield from self.wait("resident", 0, round_ & 1, round_)
            need(self.shared_item == round_, "the wrong item's K/V copied to tensor memory")
            if round_ > 0:
                last = self.first_count[round_ - 1] + self.items[round_ - 1] - 1
                need(last in self.scores_done,
                     "K/V in tensor memory replaced before the item's last scores")
            self.installed[round_] = self.installed.get(round_, 0) + 1
            self.bar["a_ready", 0].arrive()

        before = 0
        yield from install(0)
        for round_, steps in enumerate(self.items):
            for h in range(steps):
                b = h & 1
                count = before + h
                stage = count % STAGES
                yield from self.wait("scores_full", b, (count >> 1) & 1, count >> 1)
                need(count in self.scores_done and (count + 2) not in self.scores_started,
                     f"scores of sub-step {count} read while absent or overwritten")
                yield from self.wait("stage_full", stage, (count // STAGES) & 1, count // STAGES)
                need(self.stage_content[stage] == count, "statistics of the wrong sub-step read")
                yield
                need((count + 2) not in self.scores_started, "probabilities written over newer scores")
                self.written[count] = self.written.get(count, 0) + 1
                self.bar["operands_ready", b].arrive()
                yield
            before += steps
            if round_ + 1 < len(self.items):
                yield from install(round_ + 1)
            yield from self.wait("done", 0, round_ & 1, round_)
            need((before - 1) in self.grads_done, "gradients written out before the last MMAs")
            yield

    def run_tma(self):
        kind, payload = self.tma.pop(self.rng.randrange(len(self.tma)))
        if kind == "resident":
            self.shared_item = payload
            self.bar["resident", 0].arrive()
        else:
            stage, count = payload
            self.stage_content[stage] = count
            self.bar["stage_full", stage].arrive()

    def run_pipe(self):
        op = self.pipe.pop(0)
        if op[0] == "commit":
            self.bar[op[1]].arrive()
        elif op[0] == "scores":
            _, count, stage, round_ = op
            need(self.installed.get(round_, 0) == COMPUTE and round_ + 1 not in self.installed,
                 f"scores of sub-step {count} read K/V that are not (or no longer) the item's")
            need(count < 2 or (count - 2) in self.grads_done,
                 f"scores of sub-step {count} overwrite probabilities still to be read")
            self.scores_started.add(count)
            self.scores_done.add(count)
            self.stage_reads[stage] -= 1
        else:
            _, count, stage = op
            need(self.written.get(count, 0) == COMPUTE, f"gradient MMAs of {count} before all warps wrote")
            self.grads_done.add(count)
            self.stage_reads[stage] -= 1

    def run(self):
        roles = {"producer": self.producer(), "mma": self.mma_warp()}
        for index in range(COMPUTE):
            roles[f"compute{index}"] = self.compute_warp(index)
        schedule(self.rng, roles, [(self.tma, self.run_tma), (self.pipe, self.run_pipe)])
        need(not self.tma and len(self.grads_done) == sum(self.items), "work left over at the end")


BACKWARD_ITEMS = [[2], [16], [2, 2, 2], [16, 14, 2], [4, 8, 4, 2], [6, 6, 6]]


@pytest.mark.parametrize("items", BACKWARD_ITEMS, ids=[str(i) for i in BACKWARD_ITEMS])
def test_backward_protocol_holds_under_random_schedules(items):
    for seed in range(40):
        BackwardModel(items, seed).run()
