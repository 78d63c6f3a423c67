"""A randomised model of the tcgen05 kernel's mbarrier protocol, run on the CPU.

The kernel in ``tilelang_b200/csrc/umma_gemm.cuh`` is a pipeline of seven roles (two TMA
producers, two MMA issuers, two dequantising warpgroups, the epilogue) that hand ring slots to
one another through mbarriers and test them by *phase parity*. A parity test only means "the
phase I am waiting for is complete" if the phase before it is known to be complete already: a
waiter that looks at a barrier one phase too early is told "complete" for the wrong phase.
Nothing on the device reports that; the symptom is operands overwritten before the MMA has read
them, and later a hand-off that never comes.

This model copies the kernel's index arithmetic role by role (ring slots, barrier indices,
parities, who arrives where), runs the roles under a random scheduler with strongly skewed
speeds, lets TMA copies land out of order and each issuer's tensor-pipe work complete in its own
order, and checks at every wait that the phase the waiter means is the phase the barrier has
completed. It also checks ring contents (a slot overwritten before it was consumed, an MMA
reading a slot that holds another stage) and reports deadlock.

Three rules of the kernel are pinned here, each with the variant that breaks:
  * a dequantising group serves the stages of one CTA-wide parity (not "its place in the pair");
  * the depth of the tensor-memory ring is an even number of stages;
  * with one accumulator, an issuer waits for its turn before it looks at ``acc_empty``.
"""
import random

import pytest


class Violation(Exception):
    pass


class Barrier:
    """mbarrier: `count` arrivals (plus outstanding copy bytes) complete a phase."""

    def __init__(self, name, count):
        self.name, self.count, self.pending, self.completed, self.tx = name, count, count, 0, 0

    def _settle(self):
        if self.pending == 0 and self.tx == 0:
            self.completed += 1
            self.pending = self.count

    def arrive(self):
        if self.pending == 0:
            raise Violation(f"{self.name}: more arrivals than the barrier's count")
        self.pending -= 1
        self._settle()

    def arrive_expect(self, tx):
        self.tx += tx
        self.arrive()

    def complete_tx(self, tx):
        self.tx -= tx
        self._settle()

    def test(self, parity):          # mbarrier.try_wait.parity
        return (self.completed & 1) != parity


class Rings:
    """Ring depths of umma_dequant_gemm_kernel<TN, ...> (RingConfig)."""

    def __init__(self, tn, group_kblocks=None, tmem_slots=None):
        self.issuers = 2 if tn <= 128 else 1                       # issuers_for
        self.GB = 1 if tn >= 256 else (2 if tn >= 128 else 4)      # group_kblocks_for
        acc_cols = ((self.issuers * tn + 31) // 32) * 32
        self.NS = tmem_slots or (12 if (512 - acc_cols) // 32 >= 12 else 8)
        self.NBG = 6 if tn >= 256 else 4
        self.NWP = {256: 1, 128: 4, 64: 4}.get(tn, 8)       # uint4 stages; the depth depends on the format
        self.gsz = group_kblocks or self.GB                        # 1 when K is ragged


class Pipeline:
    def __init__(self, rings, segments, rng, speeds, groups_follow="stage_parity", turn_first=True):
        self.r, self.segments, self.rng, self.speeds = rings, segments, rng, speeds
        self.groups_follow, self.turn_first = groups_follow, turn_first
        r = rings
        self.full_w = [Barrier(f"full_w[{i}]", 1) for i in range(r.NWP)]
        self.empty_w = [Barrier(f"empty_w[{i}]", 8) for i in range(r.NWP)]
        self.full_b = [Barrier(f"full_b[{i}]", 1) for i in range(r.NBG)]
        self.empty_b = [Barrier(f"empty_b[{i}]", 2 if r.gsz == 4 else 1) for i in range(r.NBG)]
        self.a_full = [Barrier(f"a_full[{i}]", 4) for i in range(r.NS)]
        self.cons = [Barrier(f"cons[{i}]", 1) for i in range(r.NS // 2)]
        self.acc_full = Barrier("acc_full", r.issuers)
        self.acc_empty = Barrier("acc_empty", 4)
        self.turn = [Barrier("turn[0]", 1), Barrier("turn[1]", 1)]
        self.w_ring = [None] * r.NWP      # pair number held by each weight slot
        self.b_ring = [None] * r.NBG      # group number held by each activation slot
        self.t_ring = [None] * r.NS       # k-block held by each tensor-memory slot (None: consumed)
        self.copies = []                  # TMA copies in flight
        self.tensor_pipe = [[], []]       # per issuing thread: MMAs and commits, in order

    def wait(self, bar, parity, phase, who):
        """Blocks on the parity test; `phase` is the phase the waiter means."""
        while not bar.test(parity):
            yield (bar, parity)
        if phase >= 0 and bar.completed != phase + 1:
            raise Violation(f"{who} waits for phase {phase} of {bar.name}; the test passed with {bar.completed} phases complete")

    # ---- warp 0 ----
    def weight_producer(self):
        r, wc = self.r, 0
        for b, e in self.segments:
            for _ in range(b, e, 2):
                s = wc % r.NWP
                yield from self.wait(self.empty_w[s], ((wc // r.NWP) & 1) ^ 1, wc // r.NWP - 1, "weight producer")
                self.full_w[s].arrive_expect(1)

                def land(s=s, wc=wc):
                    self.w_ring[s] = wc
                    self.full_w[s].complete_tx(1)
                self.copies.append(("weights", land))
                wc += 1
                yield None

    # ---- warp 3 ----
    def activation_producer(self):
        r, gc = self.r, 0
        for b, e in self.segments:
            for _ in range(2 * b, 2 * e, r.gsz):
                s = gc % r.NBG
                if r.GB == 1 or (r.GB == 2 and r.gsz == 2):
                    if gc >= r.NBG:
                        prev_kb = (gc - r.NBG) * r.GB
                        yield from self.wait(self.cons[(prev_kb % r.NS) >> 1], (prev_kb // r.NS) & 1, prev_kb // r.NS,
                                             "activation producer")
                else:
                    yield from self.wait(self.empty_b[s], ((gc // r.NBG) & 1) ^ 1, gc // r.NBG - 1, "activation producer")
                self.full_b[s].arrive_expect(1)

                def land(s=s, gc=gc):
                    self.b_ring[s] = gc
                    self.full_b[s].complete_tx(1)
                self.copies.append(("activations", land))
                gc += 1
                yield None

    # ---- warps 1 and 2 ----
    def issuer(self, me):
        r = self.r
        NI, NS, NBG, GB, gsz = r.issuers, r.NS, r.NBG, r.GB, r.gsz
        g0 = gc0 = tc = my_turns = 0
        sa, pa = (2 * me) % NS, 0
        gshift, gmask = {4: 2, 2: 1, 1: 0}[gsz], gsz - 1
        queue = self.tensor_pipe[me if NI == 2 else 0]
        for b, e in self.segments:
            nst = e - b
            for i in range((me ^ g0) & 1, nst, 2):
                G = g0 + i
                grp0, grp1 = gc0 + ((2 * i) >> gshift), gc0 + ((2 * i + 1) >> gshift)
                sb0, sb1 = grp0 % NBG, grp1 % NBG
                yield from self.wait(self.a_full[sa], pa, (2 * G) // NS, f"issuer {me} (a_full)")
                yield from self.wait(self.full_b[sb0], (grp0 // NBG) & 1, grp0 // NBG, f"issuer {me} (full_b)")
                if grp1 != grp0:
                    yield from self.wait(self.full_b[sb1], (grp1 // NBG) & 1, grp1 // NBG, f"issuer {me} (full_b)")
                if i < NI and not self.turn_first:
                    yield from self.wait(self.acc_empty, (tc & 1) ^ 1, tc - 1, f"issuer {me} (acc_empty)")
                if NI == 1 and G != 0:
                    yield from self.wait(self.turn[me], my_turns & 1, my_turns, f"issuer {me} (turn)")
                    my_turns += 1
                if i < NI and self.turn_first:
                    yield from self.wait(self.acc_empty, (tc & 1) ^ 1, tc - 1, f"issuer {me} (acc_empty)")
                queue.append(("mma", G, sa, (sb0, grp0), (sb1, grp1)))
                if NI == 1:
                    self.turn[me ^ 1].arrive()
                queue.append(("commit", self.cons[sa >> 1]))
                if GB > 1 and not (GB == 2 and gsz == 2):
                    queue.append(("commit", self.empty_b[sb0]))
                    if grp1 != grp0:
                        queue.append(("commit", self.empty_b[sb1]))
                    if gsz == 4 and (i & 1) == 0 and i == nst - 1:
                        self.empty_b[sb0].arrive()
                if (i == nst - 1) if NI == 1 else (i + 2 >= nst):
                    queue.append(("commit", self.acc_full))
                sa += 4
                if sa >= NS:
                    sa, pa = sa - NS, pa ^ 1
                yield None
            if NI == 2 and nst == 1 and ((me ^ g0) & 1) != 0:
                yield from self.wait(self.acc_empty, (tc & 1) ^ 1, tc - 1, f"issuer {me} (acc_empty, idle)")
                self.acc_full.arrive()
            g0 += nst
            gc0 += (2 * nst + gmask) >> gshift
            tc += 1

    def tensor_pipe_step(self, which):
        op = self.tensor_pipe[which].pop(0)
        if op[0] == "commit":
            op[1].arrive()
            return
        _, G, sa, b0, b1 = op
        for h in range(2):
            if self.t_ring[sa + h] != 2 * G + h:
                raise Violation(f"the MMA of stage {G} reads tensor-memory slot {sa + h}, which holds k-block {self.t_ring[sa + h]}")
            self.t_ring[sa + h] = None
        for slot, grp in (b0, b1):
            if self.b_ring[slot] != grp:
                raise Violation(f"the MMA of stage {G} reads activation slot {slot}, which holds group {self.b_ring[slot]}")

    # ---- warps 4-11 ----
    def dequant_group(self, dg):
        r = self.r
        wc = kc0 = g0 = 0
        for b, e in self.segments:
            d = dg ^ (g0 & 1) if self.groups_follow == "stage_parity" else dg
            g0 += e - b
            for sti in range(b, e, 2):
                n = min(2, e - sti)
                sw = wc % r.NWP
                yield from self.wait(self.full_w[sw], (wc // r.NWP) & 1, wc // r.NWP, f"dequant group {dg} (full_w)")
                if self.w_ring[sw] != wc:
                    raise Violation(f"dequant group {dg} reads weight slot {sw}, which holds pair {self.w_ring[sw]}, not {wc}")
                if d < n:
                    for h in range(2):
                        kc = kc0 + 2 * d + h
                        sa = kc % r.NS
                        if h == 0 and kc >= r.NS:
                            prev = kc - r.NS
                            yield from self.wait(self.cons[sa >> 1], (prev // r.NS) & 1, prev // r.NS, f"dequant group {dg} (cons)")
                        if h == 1:
                            for _ in range(4):
                                self.empty_w[sw].arrive()
                            yield None
                        if self.t_ring[sa] is not None:
                            raise Violation(f"dequant group {dg} overwrites tensor-memory slot {sa} (k-block {self.t_ring[sa]} not consumed)")
                        self.t_ring[sa] = kc
                        yield None
                    for _ in range(4):
                        self.a_full[sa - 1].arrive()
                else:
                    for _ in range(4):
                        self.empty_w[sw].arrive()
                kc0 += 2 * n
                wc += 1
                yield None

    # ---- warps 12-15 ----
    def epilogue(self):
        for tc in range(len(self.segments)):
            yield from self.wait(self.acc_full, tc & 1, tc, "epilogue")
            yield None
            for _ in range(4):
                self.acc_empty.arrive()
            yield None

    def run(self, max_steps=2_000_000):
        roles = {"W": self.weight_producer(), "P": self.activation_producer(), "I0": self.issuer(0), "I1": self.issuer(1),
                 "D0": self.dequant_group(0), "D1": self.dequant_group(1), "E": self.epilogue()}
        blocked = {}
        for _ in range(max_steps):
            if not (roles or self.copies or self.tensor_pipe[0] or self.tensor_pipe[1]):
                return
            ready = [n for n in roles if blocked.get(n) is None or blocked[n][0].test(blocked[n][1])]
            kinds = {}
            for idx, (kind, _) in enumerate(self.copies):
                kinds.setdefault(kind, []).append(idx)
            ready.extend(kinds)
            ready.extend(f"pipe{q}" for q in (0, 1) if self.tensor_pipe[q])
            if not ready:
                raise Violation("deadlock: " + ", ".join(f"{n} on {blocked[n][0].name}" for n in sorted(roles)))
            x = self.rng.random() * sum(self.speeds[n] for n in ready)
            for name in ready:
                x -= self.speeds[name]
                if x <= 0:
                    break
            if name in roles:
                try:
                    blocked[name] = next(roles[name])
                except StopIteration:
                    del roles[name]
                    blocked.pop(name, None)
            elif name.startswith("pipe"):
                self.tensor_pipe_step(int(name[4]))
            else:
                self.copies.pop(self.rng.choice(kinds[name]))[1]()
        raise Violation("step limit")


def span_segments(stages_per_tile, span, cta):
    """(st_begin, st_end) of every segment of one CTA's stream-K span (SegmentWalk)."""
    pos, end, out = cta * span, (cta + 1) * span, []
    while pos < end:
        b = pos % stages_per_tile
        e = min(stages_per_tile, b + end - pos)
        out.append((b, e))
        pos += e - b
    return out


def random_span(rng, stage_counts=(1, 2, 3, 5, 8, 11, 12, 15, 16, 27, 64)):
    st = rng.choice(stage_counts)
    return span_segments(st, rng.randint(1, 6 * st + 7), rng.randint(0, 5))


ACTORS = ["W", "P", "I0", "I1", "D0", "D1", "E", "weights", "activations", "pipe0", "pipe1"]


def violations(make_rings, make_segments, runs, seed, **rules):
    found = []
    for r in range(runs):
        rng = random.Random(seed + r)
        speeds = {n: rng.choice([0.02, 0.1, 0.3, 1.0, 1.0, 3.0]) for n in ACTORS}
        try:
            Pipeline(make_rings(), make_segments(rng), rng, speeds, **rules).run()
        except Violation as v:
            found.append(str(v))
    return found


KERNELS = [(256, None), (128, None), (128, 1), (64, None), (64, 1), (32, None), (16, None)]


@pytest.mark.parametrize("tn,group_kblocks", KERNELS)
def test_every_wait_sees_the_phase_it_means(tn, group_kblocks):
    """Random spans (whole tiles, cut tiles, odd and even stage counts, one-stage tiles)."""
    found = violations(lambda: Rings(tn, group_kblocks), random_span, runs=150, seed=1000 * tn)
    assert not found, found[0]


@pytest.mark.parametrize("tn,weight_pairs,activation_groups", [(256, 2, 5), (128, 1, 4), (128, 3, 4), (64, 2, 4), (16, 3, 4)])
def test_other_ring_depths(tn, weight_pairs, activation_groups):
    """Other formats have larger stages and so shallower shared-memory rings (int4 -> int8: five
    activation groups at the 256-token tile)."""
    def rings():
        r = Rings(tn)
        r.NWP, r.NBG = weight_pairs, activation_groups
        return r
    found = violations(rings, random_span, runs=100, seed=31 * tn + weight_pairs)
    assert not found, found[0]


@pytest.mark.parametrize("tn", [128, 64, 32])
def test_many_tiles_with_an_odd_stage_count(tn):
    """The schedule that exposed the flaw: tens of short tiles per CTA, 11 stages each."""
    found = violations(lambda: Rings(tn), lambda rng: [(0, 11)] * 40, runs=60, seed=7)
    assert not found, found[0]


def test_groups_that_follow_their_place_in_the_pair_are_caught():
    """After a segment with an odd number of stages the groups swap issuers; a group then waits on a
    `cons` barrier it last saw two phases ago and can pass one phase early."""
    found = violations(lambda: Rings(128), lambda rng: [(0, 11)] * 40, runs=60, seed=7, groups_follow="pair_position")
    assert any("dequant group" in v and "cons" in v for v in found)
    # with an even stage count nothing swaps, which is why that schedule never failed
    assert not violations(lambda: Rings(128), lambda rng: [(0, 12)] * 40, runs=60, seed=7, groups_follow="pair_position")


def test_an_odd_ring_depth_in_stages_is_caught():
    """14 slots = 7 stages: a stage returns to a barrier last used by a stage of the other parity."""
    found = violations(lambda: Rings(32, tmem_slots=14), lambda rng: [(0, 12)] * 40, runs=60, seed=7)
    assert any("cons" in v for v in found)


def test_acc_empty_before_turn_is_caught_with_one_stage_tiles():
    found = violations(lambda: Rings(256), lambda rng: [(0, 1)] * 20, runs=60, seed=7, turn_first=False)
    assert any("acc_empty" in v for v in found)
    assert not violations(lambda: Rings(256), lambda rng: [(0, 1)] * 20, runs=60, seed=7, turn_first=True)
