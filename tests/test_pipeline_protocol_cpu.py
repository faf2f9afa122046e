"""The large-M kernel's barrier protocol, model-checked on the host under random schedules (no GPU)."""
import dataclasses
import random

import pytest

from pipeline_model import Pipeline, ProtocolError, config_from_source


@pytest.mark.parametrize('tm', [256, 64])
def test_kernel_configuration_is_consistent(tm):
    cfg = config_from_source(tm)
    assert cfg.group_warps * cfg.conv_groups == 8
    # the (slot, group) pair of stage i is (i % raw_slots, i % conv_groups): it recurs with the least common multiple
    lcm = next(n for n in range(1, 1000) if n % cfg.raw_slots == 0 and n % cfg.conv_groups == 0)
    assert cfg.raw_period == lcm
    # a group converting a stage needs its int8 slot and its f16 slot at once, and the ring must hold the
    # stages under conversion plus the ones the tensor core works on
    assert cfg.stages >= cfg.conv_groups + 2 or cfg.stages >= 4
    assert cfg.raw_slots >= cfg.conv_groups or cfg.raw_slots >= 3


@pytest.mark.parametrize('tm', [256, 64])
@pytest.mark.parametrize('tiles,k_blocks', [(1, 1), (1, 7), (3, 8), (5, 13), (2, 64)])
def test_protocol_holds_under_random_schedules(tm, tiles, k_blocks):
    cfg = config_from_source(tm)
    for seed in range(40):
        for delay in (0.2, 0.9, 0.99):   # copies land promptly ... copies land very late and far out of order
            Pipeline(cfg, tiles, k_blocks, random.Random(seed)).run(copy_delay=delay)


def test_model_catches_a_shared_barrier_for_slots_that_change_groups():
    """Three int8 slots taken in turn by two converter groups with ONE barrier per slot: a group that skipped a use
    of a slot takes the pending phase of the other group's copy for its own.  The model must find that."""
    cfg = dataclasses.replace(config_from_source(256), per_group_barriers=False)
    assert cfg.raw_slots % cfg.conv_groups != 0
    failures = 0
    for seed in range(60):
        try:
            Pipeline(cfg, 3, 16, random.Random(seed)).run(copy_delay=0.9)
        except ProtocolError:
            failures += 1
    assert failures > 0


def test_shared_barrier_is_fine_when_every_slot_keeps_its_group():
    cfg = dataclasses.replace(config_from_source(64), per_group_barriers=False)
    assert cfg.raw_slots % cfg.conv_groups == 0
    for seed in range(30):
        Pipeline(cfg, 3, 16, random.Random(seed)).run(copy_delay=0.9)


@pytest.mark.parametrize('tm', [256, 64])
def test_a_wait_that_runs_out_ends_every_role_and_the_cta_retires_clean(tm):
    """Any role's wait may run out at any time (modelled: the n-th time the scheduler finds that role blocked).  The
    role raises the CTA-wide flag, every other wait ends on it, the producer waits for the copies it armed and the
    MMA lane for a final commit: when the last role is gone nothing is in flight, so nothing writes to shared
    memory or reads tensor memory of a CTA that has retired."""
    cfg = config_from_source(tm)
    n_agents = 2 + 8 + 4
    runs = 0
    for seed in range(25):
        for agent in range(n_agents):
            for nth in (1, 3, 17):
                pipe = Pipeline(cfg, 3, 9, random.Random(seed))
                pipe.expire = (agent, nth)
                pipe.run(copy_delay=0.9)
                runs += 1 if pipe.abort else 0
    assert runs > 100   # the flag was really raised in most of these schedules


def test_model_catches_a_teardown_without_the_drain():
    cfg = dataclasses.replace(config_from_source(256), drain_on_exit=False)
    failures = 0
    for seed in range(40):
        pipe = Pipeline(cfg, 3, 9, random.Random(seed))
        pipe.expire = (1, 2)   # the MMA lane gives up early: copies and commits are still in flight
        try:
            pipe.run(copy_delay=0.95)
        except ProtocolError as e:
            assert 'retired with' in str(e)
            failures += 1
    assert failures > 0
