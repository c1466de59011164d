"""The inbox protocol of the push collectives, run as CPU threads (csrc/comm/protocol_model.cpp): sentinel-carrying
units whose words land in any order, the three-slot rotation with its re-arm-the-previous-slot rule, the fused linear's
slot pairs re-armed by their readers, bounded waits.  Ranks are delayed at random; every result is compared with the
exact sum.  A lost message must show on every rank and recovery must restore exact results."""
import ctypes as C

import pytest

from agens_engine_b200 import _lib


def _run(ranks, calls, max_units, seed, mode=0, lose_rank=-1, lose_call=-1, timeout_ms=20000):
    h = _lib.host_lib()
    fn = h.b2h_comm_model_run
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_uint, C.c_int, C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_int]
    rep = C.create_string_buffer(256)
    rc = fn(ranks, calls, max_units, seed, mode, lose_rank, lose_call, timeout_ms, rep, 256)
    return rc, rep.value.decode()


@pytest.mark.parametrize("ranks", [1, 2, 3, 4, 8])
def test_rotating_calls_stay_exact_under_random_delays(ranks):
    for seed in range(4):
        rc, rep = _run(ranks, 150, 24, seed)
        assert rc == 0, rep


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_fused_linear_slot_pairs(ranks):
    for seed in range(3):
        rc, rep = _run(ranks, 90, 16, 100 + seed, mode=1)
        assert rc == 0, rep


@pytest.mark.parametrize("ranks,lose_rank", [(2, 1), (4, 0), (4, 3)])
def test_a_lost_message_times_out_everywhere_and_recovery_restores_exact_results(ranks, lose_rank):
    rc, rep = _run(ranks, 40, 8, 7, lose_rank=lose_rank, lose_call=17, timeout_ms=300)
    assert rc == 0 and f"ranks_that_saw_the_loss {ranks}" in rep, rep


def test_arguments_are_checked():
    assert _run(9, 10, 8, 0)[0] == -1 and _run(2, 0, 8, 0)[0] == -1 and _run(2, 10, 0, 0)[0] == -1


def test_a_two_slot_rotation_is_caught():
    """The model must have teeth: with two slots a call re-arms the slot that a faster peer is already writing for the
    next call, which shows as a message that never arrives."""
    caught = 0
    for seed in range(6):
        rc, rep = _run(4, 14, 24, seed, mode=2, timeout_ms=100)
        caught += rc != 0
    assert caught >= 3
