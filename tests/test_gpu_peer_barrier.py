"""The bounded completion barrier of the fused exchanges, on one GPU: a wait whose flag nobody sets
runs out, reports GK_DEV_WAIT_EXPIRED through the status word and leaves the context usable; a wait
whose flags are already there passes.  (Two ranks signalling each other are covered by the 2-GPU
test; two kernels waiting for one another are never launched on one GPU.)"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHORT = 2_000_000          # cycles: about a millisecond


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


def test_wait_runs_out_and_is_reported(rt):
    mine, peer = torch.zeros(8, dtype=torch.int32, device=DEV), torch.zeros(8, dtype=torch.int32, device=DEV)
    assert rt._C._take_device_status() == 0
    torch.ops.gaudirt._peer_barrier([mine, peer], 0, 1, SHORT)          # rank 0 of 2; "rank 1" never signals
    assert rt._C._take_device_status() == 4                              # GK_DEV_WAIT_EXPIRED, then cleared
    assert rt._C._take_device_status() == 0
    assert mine.tolist()[:2] == [1, 0] and peer.tolist()[:2] == [1, 0]   # its own signal went out to both arrays
    # the context is intact: ordinary work runs afterwards
    assert float(torch.ones(1000, device=DEV).sum()) == 1000.0


def test_flags_already_there_let_it_pass(rt):
    mine, peer = torch.zeros(8, dtype=torch.int32, device=DEV), torch.zeros(8, dtype=torch.int32, device=DEV)
    mine[1] = 5                                                          # the peer's epoch-5 signal has landed
    torch.ops.gaudirt._peer_barrier([mine, peer], 0, 5, SHORT)
    assert rt._C._take_device_status() == 0 and peer.tolist()[0] == 5
    mine[1] = 9                                                          # epochs only grow: a later one also satisfies 6
    torch.ops.gaudirt._peer_barrier([mine, peer], 0, 6, SHORT)
    assert rt._C._take_device_status() == 0


def test_counted_form_keeps_its_epoch_on_the_device(rt):
    mine, peer = torch.zeros(8, dtype=torch.int32, device=DEV), torch.zeros(8, dtype=torch.int32, device=DEV)
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    mine[1] = 2
    for expected in (1, 2):                                              # two launches, no host-side epoch
        torch.ops.gaudirt._peer_barrier_counted([mine, peer], 0, counter, SHORT)
        assert counter.item() == expected and peer.tolist()[0] == expected
    assert rt._C._take_device_status() == 0
    torch.ops.gaudirt._peer_barrier_counted([mine, peer], 0, counter, SHORT)   # epoch 3 > the peer's 2: runs out
    assert counter.item() == 3 and rt._C._take_device_status() == 4
    with pytest.raises(RuntimeError, match="epoch counter"):
        torch.ops.gaudirt._peer_barrier_counted([mine, peer], 0, torch.zeros(2, dtype=torch.int32, device=DEV), SHORT)


def test_step_end_check_raises_when_a_wait_ran_out(rt):
    """The exchanges hand out their buffers even when the bounded wait expired (the kernel only sets a status bit);
    the step-end check is what turns that into an error instead of an incomplete activation."""
    from gaudirt_b200 import tp
    mine, peer = torch.zeros(8, dtype=torch.int32, device=DEV), torch.zeros(8, dtype=torch.int32, device=DEV)
    tp.check_device_status(DEV)                                          # clean: no raise
    torch.ops.gaudirt._peer_barrier([mine, peer], 0, 1, SHORT)           # the peer never signals
    with pytest.raises(RuntimeError, match="bounded wait ran out"):
        tp.check_device_status(DEV)
    tp.check_device_status(DEV)                                          # the word was cleared by the failed check
