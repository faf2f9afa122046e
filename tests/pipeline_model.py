"""A host-side model of the large-M kernel's producer / converter / MMA / epilogue pipeline.

The kernel (hidet_b200/csrc/qlinear_prefill.cu) synchronises its warps with mbarriers waited on by phase
parity.  A parity wait cannot tell a phase from the one two steps away, so the protocol is only correct if
no waiter can ever be two phases off.  This model restates the protocol (which barrier each role waits on,
with which parity, and what it signals), runs it under randomly interleaved schedules in which copies land
out of order and late, and checks that every role only ever touches the data it means to touch and that
nothing stalls.  Ring depths and group counts are read from the kernel source.

Test infrastructure only.
"""
from __future__ import annotations

import os
import random
import re
from dataclasses import dataclass
from typing import Callable, Dict, Generator, List, Optional, Tuple

KERNEL_SOURCE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'hidet_b200', 'csrc', 'qlinear_prefill.cu')


class ProtocolError(AssertionError):
    pass


@dataclass
class PipelineConfig:
    stages: int          # f16 weight + activation ring
    raw_slots: int       # int8 ring
    conv_groups: int     # converter groups taking stages in turn
    group_warps: int
    raw_period: int      # stages after which a (slot, group) pair recurs
    per_group_barriers: bool = True   # one "landed" barrier per (slot, group); False = one per slot
    drain_on_exit: bool = True        # producer / MMA lane wait for what they have in flight before the CTA retires


def _ternary(text: str, name: str, tm: int) -> int:
    m = re.search(r'static constexpr int %s = TM == 256 \? (\d+) : (\d+);' % name, text)
    if m is None:
        raise ProtocolError('cannot find {} in the kernel source'.format(name))
    return int(m.group(1) if tm == 256 else m.group(2))


def config_from_source(tm: int) -> PipelineConfig:
    text = open(KERNEL_SOURCE).read()
    conv_warps = int(re.search(r'constexpr int CONV_WARPS = (\d+);', text).group(1))
    groups = _ternary(text, 'CONV_GROUPS', tm)
    return PipelineConfig(stages=_ternary(text, 'STAGES', tm), raw_slots=_ternary(text, 'RAW_SLOTS', tm), conv_groups=groups,
                          group_warps=conv_warps // groups, raw_period=_ternary(text, 'RAW_PERIOD', tm))


class Barrier:
    """mbarrier: a phase completes when the expected arrivals have come and no copy bytes are outstanding."""

    def __init__(self, name: str, count: int):
        self.name, self.count = name, count
        self.arrived = 0
        self.tx = 0
        self.phases_done = 0

    def _settle(self):
        if self.arrived == self.count and self.tx == 0:
            self.arrived = 0
            self.phases_done += 1

    def arrive(self):
        if self.arrived >= self.count:
            raise ProtocolError('{}: more arrivals than the phase expects'.format(self.name))
        self.arrived += 1
        self._settle()

    def arrive_expect_tx(self, n: int):
        if self.arrived >= self.count:
            raise ProtocolError('{}: a second copy armed on a phase that is still pending'.format(self.name))
        self.tx += n
        self.arrived += 1

    def complete_tx(self, n: int):
        self.tx -= n
        self._settle()

    def test(self, parity: int) -> bool:
        """try_wait.parity: true when the phase of that parity is not the one in progress."""
        return (self.phases_done & 1) != (parity & 1)


Wait = Optional[Callable[[], bool]]


class Aborted(Exception):
    """Raised inside a role when the CTA-wide abort flag ends one of its waits."""


class Pipeline:
    def __init__(self, cfg: PipelineConfig, tiles: int, k_blocks: int, rng: random.Random):
        self.cfg, self.tiles, self.k_blocks, self.rng = cfg, tiles, k_blocks, rng
        c = cfg
        if c.per_group_barriers:
            self.raw_full = [[Barrier('raw_full[{}][{}]'.format(r, g), 1) for g in range(c.conv_groups)] for r in range(c.raw_slots)]
        else:
            shared = [Barrier('raw_full[{}]'.format(r), 1) for r in range(c.raw_slots)]
            self.raw_full = [[shared[r]] * c.conv_groups for r in range(c.raw_slots)]
        self.raw_empty = [Barrier('raw_empty[{}]'.format(r), c.group_warps) for r in range(c.raw_slots)]
        self.act_full = [Barrier('act_full[{}]'.format(s), 1) for s in range(c.stages)]
        self.conv_full = [Barrier('conv_full[{}]'.format(s), c.group_warps) for s in range(c.stages)]
        self.slot_free = [Barrier('slot_free[{}]'.format(s), 1) for s in range(c.stages)]
        self.acc_full = [Barrier('acc_full[{}]'.format(b), 1) for b in range(2)]
        self.acc_empty = [Barrier('acc_empty[{}]'.format(b), 4) for b in range(2)]
        # what each buffer holds: the stage index (or tile index) whose data is in it
        self.raw_content: List[Optional[int]] = [None] * c.raw_slots
        self.act_content: List[Optional[int]] = [None] * c.stages
        self.conv_content: List[Dict[int, int]] = [dict() for _ in range(c.stages)]   # warp -> stage index it wrote
        self.acc_content: List[Optional[Tuple[str, int]]] = [None, None]
        self.copies: List[Callable[[], None]] = []      # copies in flight: may land in any order
        self.commits: List[Callable[[], None]] = []     # tensor-core commits: land in order
        self.mma_reading: Dict[int, int] = {}           # stage slot -> stage index the tensor core still reads
        self.abort = False                              # the CTA-wide flag a role raises when its own wait runs out
        self.expire: Optional[Tuple[int, int]] = None   # (agent, n): that agent's n-th blocked wait "runs out"
        self.retired_dirty: Optional[str] = None

    # ---- roles ----
    def producer(self) -> Generator[Wait, None, None]:
        try:
            yield from self._producer_loop()
        except Aborted:
            pass
        if self.cfg.drain_on_exit:
            # teardown: every copy armed by this lane must have landed (copies land without anyone's help)
            yield ('drain', lambda: not self.copies)

    def _producer_loop(self) -> Generator[Wait, None, None]:
        c = self.cfg
        i = 0
        for _tile in range(self.tiles):
            for _kb in range(self.k_blocks):
                r, use_r = i % c.raw_slots, i // c.raw_slots
                if use_r >= 1:
                    yield lambda r=r, p=(use_r - 1) & 1: self.raw_empty[r].test(p)
                bar = self.raw_full[r][i % c.conv_groups]
                bar.arrive_expect_tx(1)

                def land_raw(r=r, i=i, bar=bar):
                    self.raw_content[r] = i
                    bar.complete_tx(1)

                self.copies.append(land_raw)
                yield None
                s, use = i % c.stages, i // c.stages
                if use >= 1:
                    yield lambda s=s, p=(use - 1) & 1: self.slot_free[s].test(p)
                self.act_full[s].arrive_expect_tx(1)

                def land_act(s=s, i=i):
                    if s in self.mma_reading:
                        raise ProtocolError('activation tile {} lands in a slot the tensor core still reads'.format(i))
                    self.act_content[s] = i
                    self.act_full[s].complete_tx(1)

                self.copies.append(land_act)
                yield None
                i += 1

    def converter(self, group: int, warp: int) -> Generator[Wait, None, None]:
        try:
            yield from self._converter_loop(group, warp)
        except Aborted:
            pass

    def _converter_loop(self, group: int, warp: int) -> Generator[Wait, None, None]:
        c = self.cfg
        for i in range(self.tiles * self.k_blocks):
            if i % c.conv_groups != group:
                continue
            r, use_r = i % c.raw_slots, i // c.raw_slots
            s, use = i % c.stages, i // c.stages
            parity = (i // c.raw_period) & 1 if c.per_group_barriers else use_r & 1
            yield lambda r=r, p=parity: self.raw_full[r][group].test(p)
            if use >= 1:
                yield lambda s=s, p=(use - 1) & 1: self.slot_free[s].test(p)
            if self.raw_content[r] != i:
                raise ProtocolError('converter group {} reads slot {} for stage {} but it holds {}'.format(group, r, i, self.raw_content[r]))
            yield None
            self.raw_empty[r].arrive()
            yield None
            if s in self.mma_reading:
                raise ProtocolError('converter writes stage slot {} while the tensor core reads it'.format(s))
            self.conv_content[s][warp] = i
            self.conv_full[s].arrive()
            yield None

    def mma(self) -> Generator[Wait, None, None]:
        try:
            yield from self._mma_loop()
        except Aborted:
            pass
        if self.cfg.drain_on_exit:
            # teardown: a final commit; it arrives when every MMA issued so far has completed
            yield ('drain', lambda: not self.commits)

    def _mma_loop(self) -> Generator[Wait, None, None]:
        c = self.cfg
        i = 0
        for t in range(self.tiles):
            buf, acc_use = t & 1, t >> 1
            if acc_use >= 1:
                yield lambda buf=buf, p=(acc_use - 1) & 1: self.acc_empty[buf].test(p)
            self.acc_content[buf] = ('writing', t)
            for _kb in range(self.k_blocks):
                s, use = i % c.stages, i // c.stages
                yield lambda s=s, p=use & 1: self.act_full[s].test(p)
                yield lambda s=s, p=use & 1: self.conv_full[s].test(p)
                wrote = self.conv_content[s]
                if self.act_content[s] != i or len(wrote) != c.group_warps or any(v != i for v in wrote.values()):
                    raise ProtocolError('MMA of stage {} finds activations {} and weights {}'.format(i, self.act_content[s], wrote))
                self.mma_reading[s] = i

                def done(s=s, i=i):
                    if self.act_content[s] != i:
                        raise ProtocolError('stage {} was overwritten under the tensor core'.format(i))
                    del self.mma_reading[s]
                    self.conv_content[s] = dict()
                    self.slot_free[s].arrive()

                self.commits.append(done)
                yield None
                i += 1

            def finished(buf=buf, t=t):
                self.acc_content[buf] = ('done', t)
                self.acc_full[buf].arrive()

            self.commits.append(finished)
            yield None

    def epilogue(self, warp: int) -> Generator[Wait, None, None]:
        try:
            yield from self._epilogue_loop(warp)
        except Aborted:
            pass

    def _epilogue_loop(self, _warp: int) -> Generator[Wait, None, None]:
        for t in range(self.tiles):
            buf, acc_use = t & 1, t >> 1
            yield lambda buf=buf, p=acc_use & 1: self.acc_full[buf].test(p)
            if self.acc_content[buf] != ('done', t):
                raise ProtocolError('epilogue of tile {} reads an accumulator holding {}'.format(t, self.acc_content[buf]))
            yield None
            if self.acc_content[buf] != ('done', t):
                raise ProtocolError('accumulator of tile {} was overwritten while being read'.format(t))
            self.acc_empty[buf].arrive()
            yield None

    # ---- scheduler ----
    def run(self, copy_delay: float = 0.5, max_steps: int = 2_000_000) -> int:
        """Runs all roles to completion under a random schedule; returns the number of steps taken.
        `copy_delay` is the chance that a step is not spent on landing a copy even though one is in flight."""
        c = self.cfg
        agents: List[Generator[Wait, None, None]] = [self.producer(), self.mma()]
        agents += [self.converter(g, w) for g in range(c.conv_groups) for w in range(c.group_warps)]
        agents += [self.epilogue(w) for w in range(4)]
        waits: List = [None] * len(agents)
        alive = [True] * len(agents)
        blocked_count = [0] * len(agents)
        steps = 0

        def ready(k: int) -> bool:
            w = waits[k]
            if w is None:
                return True
            if isinstance(w, tuple):          # a teardown wait: not cut short by the abort flag
                return w[1]()
            if w():
                return True
            if self.abort:
                return True                   # the wait ends; the role sees the flag and leaves
            return False

        while any(alive) or self.copies or self.commits:
            steps += 1
            if steps > max_steps:
                raise ProtocolError('no end after {} steps'.format(max_steps))
            if not any(alive) and (self.copies or self.commits) and self.retired_dirty is None:
                self.retired_dirty = '{} copies and {} commits in flight'.format(len(self.copies), len(self.commits))
            # a blocked wait of the chosen agent "runs out": that role raises the flag
            if self.expire is not None and not self.abort:
                k, n = self.expire
                if alive[k] and waits[k] is not None and not isinstance(waits[k], tuple) and not waits[k]():
                    blocked_count[k] += 1
                    if blocked_count[k] >= n:
                        self.abort = True
            runnable = [k for k in range(len(agents)) if alive[k] and ready(k)]
            choices: List[Tuple[str, int]] = [('agent', k) for k in runnable]
            if self.commits:
                choices.append(('commit', 0))
            if self.copies and (not choices or self.rng.random() > copy_delay):
                choices.append(('copy', self.rng.randrange(len(self.copies))))
            if not choices:
                stuck = [k for k in range(len(agents)) if alive[k]]
                raise ProtocolError('deadlock: roles {} wait and nothing is in flight'.format(stuck))
            kind, k = self.rng.choice(choices)
            if kind == 'copy':
                self.copies.pop(k)()
            elif kind == 'commit':
                self.commits.pop(0)()
            else:
                try:
                    w = waits[k]
                    if w is not None and not isinstance(w, tuple) and self.abort and not w():
                        waits[k] = agents[k].throw(Aborted())   # the wait ended because of the flag
                    else:
                        waits[k] = next(agents[k])
                except StopIteration:
                    alive[k] = False
        if self.retired_dirty is not None:
            raise ProtocolError('the CTA retired with ' + self.retired_dirty)
        return steps
