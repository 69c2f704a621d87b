"""Status mailbox of the peer-memory kernels: failures of an earlier step surface at the next call without a
host synchronisation, the words are cleared between steps, and a failure callback runs before the error."""
import pytest
import torch

from apexw_b200.parallel.status import PeerStepError, StatusMailbox, ZS_ENTRY_TIMEOUT, ZS_EXIT_TIMEOUT


def test_clean_posts_raise_nothing_and_recycle_their_slots():
    box = StatusMailbox(torch.device("cpu"), words=4, depth=2)
    for _ in range(7):                      # more posts than host slots
        box.post()
        box.poll("unit", 0)
    assert box.read_now() == [0, 0, 0, 0]


def test_failure_is_reported_once_with_its_word_and_the_callback_runs_first():
    box = StatusMailbox(torch.device("cpu"), words=3)
    seen = []
    box.word(1).fill_(ZS_ENTRY_TIMEOUT)
    box.post(lambda codes: seen.append(dict(codes)))
    assert box.read_now() == [0, 0, 0]      # cleared for the next step
    with pytest.raises(PeerStepError) as err:
        box.poll("unit step", 3)
    assert seen == [{1: ZS_ENTRY_TIMEOUT}] and err.value.codes == {1: ZS_ENTRY_TIMEOUT}
    assert "rank 3" in str(err.value) and "nothing was updated" in str(err.value)
    box.poll("unit step", 3)                # reported once
    box.word(7).fill_(ZS_EXIT_TIMEOUT)      # indices past the end share the last word
    box.post()
    with pytest.raises(RuntimeError):
        box.poll("unit step", 3, wait=True)


def test_several_pending_posts_are_folded_oldest_first():
    box = StatusMailbox(torch.device("cpu"), words=2, depth=2)
    order = []
    box.word(0).fill_(ZS_EXIT_TIMEOUT)
    box.post(lambda c: order.append("first"))
    box.post(lambda c: order.append("second"))          # clean: its callback must not run
    box.word(1).fill_(ZS_ENTRY_TIMEOUT)
    box.post(lambda c: order.append("third"))           # forces the oldest post to be folded in (two slots only)
    with pytest.raises(PeerStepError) as err:
        box.poll()
    assert order == ["first", "third"] and err.value.codes == {0: ZS_EXIT_TIMEOUT, 1: ZS_ENTRY_TIMEOUT}
