"""Host model of the cross-GPU flag protocols (CPU threads over atomics, randomised delays): the rules the kernels
use hold, and the model catches the variants that break them."""
import pytest

from hotspa_ae_b200 import core as C


@pytest.mark.parametrize("n,first_epoch", [(2, 1), (4, 1), (8, 1), (4, 2 ** 32 - 50)])
def test_barrier_epochs_including_wrap_around(n, first_epoch):
    r = C.run_barrier_model(n, 200, first_epoch, seed=n)
    assert r["checks"] == 200 * n * n and r["violations"] == 0 and r["timeouts"] == 0, r


@pytest.mark.parametrize("n", [2, 4, 8])
def test_reduce_scatter_three_counter_sets_two_receive_buffers(n):
    r = C.run_reduce_scatter_model(n, 150, 3, 2, 4, 4, seed=7 + n)
    assert r["violations"] == 0 and r["timeouts"] == 0 and r["checks"] == 150 * n * 4 * n * 5, r


def test_reduce_scatter_variants_that_break_are_caught():
    # two counter sets: the set cleared at the start of a call is the one its peers are adding into -> lost counts
    r = C.run_reduce_scatter_model(4, 100, 2, 2, 4, 4, seed=1)
    assert r["violations"] + r["timeouts"] > 0, r
    # one receive buffer: a fast peer's next call overwrites parts that are still being reduced
    r = C.run_reduce_scatter_model(4, 150, 3, 1, 4, 4, seed=2)
    assert r["violations"] > 0, r


@pytest.mark.parametrize("n", [2, 4, 8])
def test_all_gather_two_staging_buffers(n):
    r = C.run_all_gather_model(n, 200, 2, 8, seed=11 + n)
    assert r["violations"] == 0 and r["timeouts"] == 0 and r["checks"] == 200 * n * (n - 1) * 8, r


def test_all_gather_single_staging_buffer_is_caught():
    r = C.run_all_gather_model(4, 300, 1, 8, seed=3)
    assert r["violations"] > 0, r
