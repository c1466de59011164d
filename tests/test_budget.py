"""Memory-budget ledger and plan-driven sizing (CPU): refusal past the budget with a fake allocator, pool / context /
tier decisions from the planner, minimum over ranks (reference: crates/agens-cli/src/m1.rs:492-541, 905-974,
plan.rs:182-241, tp.rs:77-90)."""
import pytest

from agens_engine_b200.models import config as C
from agens_engine_b200.serve import budget as B


def test_ledger_refuses_past_the_budget_and_keeps_books():
    led = B.BudgetLedger(10 * B.GiB)
    made = []

    def fake_alloc(n):
        def go():
            made.append(n)
            return object()
        return go

    led.alloc("weights", 6 * B.GiB, fake_alloc(6))
    led.alloc("kv", 3 * B.GiB, fake_alloc(3))
    with pytest.raises(B.BudgetExceeded) as e:
        led.alloc("scratch", 2 * B.GiB, fake_alloc(2))
    assert "scratch" in str(e.value) and made == [6, 3]          # the refused allocation was never attempted
    assert led.used == 9 * B.GiB and led.free() == B.GiB
    led.release("kv")
    led.alloc("scratch", 2 * B.GiB, fake_alloc(2))
    assert made == [6, 3, 2]

    def failing():
        raise MemoryError("device says no")
    with pytest.raises(MemoryError):
        led.alloc("more", B.GiB, failing)
    assert "more" not in led.items                                # a failed allocation leaves no booking behind
    assert any("total" in line for line in led.report())


def test_unlimited_ledger_only_reports():
    led = B.BudgetLedger(0)
    led.book("x", 500 * B.GiB)
    assert led.free() > 0 and "no cap" in led.report()[-1]


def test_plan_sizes_pool_context_and_tier():
    cfg = C.dense_32b(seed=0)
    # a roomy budget: everything on the GPU, the pool is not larger than every slot at full context
    big = B.plan_deployment(cfg, 160, 8192, 16, 16, 2048, tp=1, gpu_free_gib=170, host_avail_gib=64)
    assert big.fits and not big.host_tier and big.max_ctx == 8192
    assert big.n_pages == (8192 // 16) * 16
    # 24 GiB: the weights fit, a 262,148-token context does not: the tier goes to the host and the context stays whole
    mid = B.plan_deployment(cfg, 24, 262148, 1, 1, 2048, tp=1, gpu_free_gib=170, host_avail_gib=200)
    assert mid.fits and mid.host_tier and mid.max_ctx == 262148 and 0 < mid.n_pages < 262148 // 16
    # the same without host memory: the context is clamped to what the pool holds, not refused
    clamp = B.plan_deployment(cfg, 24, 262148, 1, 1, 2048, tp=1, gpu_free_gib=170, host_avail_gib=0)
    assert clamp.fits and clamp.max_ctx < 262148 and clamp.max_ctx == clamp.plan["context"]
    # 16 GiB on one GPU: the weights alone do not fit; on four GPUs they do
    assert not B.plan_deployment(cfg, 16, 262148, 1, 1, 2048, tp=1, gpu_free_gib=170, host_avail_gib=200).fits
    tp4 = B.plan_deployment(cfg, 16, 262148, 1, 1, 2048, tp=4, gpu_free_gib=170, host_avail_gib=200)
    assert tp4.fits and tp4.n_pages > 0
    assert any("plan:" in line for line in tp4.lines)


def test_ranks_take_the_minimum():
    cfg = C.dense_32b(seed=0)
    a = B.plan_deployment(cfg, 24, 65536, 4, 4, 2048, tp=2, gpu_free_gib=170, host_avail_gib=64)
    other = [a.n_pages - 100, a.max_ctx - 64, a.resident_window_tokens, 1]

    def all_min(v):
        if len(v) == 4:
            return [min(x, y) for x, y in zip(v, other)]
        return [0]                                    # some rank needs the host tier
    m = B.agree_min(a, all_min)
    assert m.n_pages == a.n_pages - 100 and m.max_ctx == a.max_ctx - 64 and m.host_tier
