"""Self-tests of the trace verifier: hand-written traces that are right, and traces with one planted defect each
(a missing wait, a wait nobody posts, a cycle, an access outside a buffer, a write into a user input, a contribution
reduced twice, a missing contribution).  The verifier has to accept the first kind and name the defect of the second."""
import ctypes

from hccl_b200._lib import lib


def verify(script: str) -> str:
    lib.HcclDebugVerifyTrace.restype = ctypes.c_int
    lib.HcclDebugVerifyTrace.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32]
    buf = ctypes.create_string_buffer(1 << 14)
    rc = lib.HcclDebugVerifyTrace(script.strip().encode(), buf, len(buf))
    assert rc == 0, rc
    return buf.value.decode()


# two ranks, four fp32 elements: each rank copies its input to its output, tells the peer, then adds the peer's input
GOOD_ALLREDUCE = """
ranks 2 op allreduce count 4
0 0 copy 0:out:0 0:in:0 16
0 0 post 1 0
0 0 wait 1 0
0 0 reduce 0:out:0 1:in:0 16
1 0 copy 1:out:0 1:in:0 16
1 0 post 0 0
1 0 wait 0 0
1 0 reduce 1:out:0 0:in:0 16
"""


def test_correct_traces_pass():
    rep = verify(GOOD_ALLREDUCE)
    assert rep.startswith("OK: 8 tasks (4 data)"), rep
    gather = """
ranks 2 op allgather count 2
0 0 copy 0:out:0 0:in:0 8
0 0 copy 0:out:8 1:in:0 8
1 0 copy 1:out:8 1:in:0 8
1 0 copy 1:out:0 0:in:0 8
"""
    assert verify(gather).startswith("OK"), verify(gather)


def test_missing_synchronisation_is_a_memory_conflict():
    # rank 1 writes into rank 0's output while rank 0 may still be copying into it: nothing orders the two
    racy = """
ranks 2 op allreduce count 4
0 0 copy 0:out:0 0:in:0 16
1 0 copy 1:out:0 1:in:0 16
1 0 reduce 0:out:0 1:in:0 16
0 0 reduce 1:out:0 0:in:0 16
"""
    rep = verify(racy)
    assert rep.startswith("FAILED") and "unordered accesses to rank" in rep, rep


def test_unmatched_wait_and_stale_post():
    hang = GOOD_ALLREDUCE.replace("1 0 post 0 0\n", "")
    rep = verify(hang)
    assert rep.startswith("FAILED") and "would hang" in rep, rep
    stale = GOOD_ALLREDUCE + "0 0 post 1 3\n"
    rep = verify(stale)
    assert rep.startswith("FAILED") and "stale post" in rep, rep


def test_cycle_is_a_deadlock():
    # both ranks wait for the other before they post
    cyc = """
ranks 2 op allreduce count 4
0 0 wait 1 0
0 0 post 1 0
1 0 wait 0 0
1 0 post 0 0
"""
    rep = verify(cyc)
    assert rep.startswith("FAILED") and "deadlock" in rep, rep


def test_bounds_and_input_writes():
    oob = GOOD_ALLREDUCE.replace("0 0 copy 0:out:0 0:in:0 16", "0 0 copy 0:out:8 0:in:0 16")
    rep = verify(oob)
    assert rep.startswith("FAILED") and "leaves its buffer" in rep, rep
    clobber = GOOD_ALLREDUCE + "0 0 copy 0:in:0 0:out:0 16\n"
    rep = verify(clobber)
    assert rep.startswith("FAILED") and "writes a user input buffer" in rep, rep


def test_semantic_defects():
    twice = GOOD_ALLREDUCE + "0 0 reduce 0:out:0 0:in:0 16\n"
    rep = verify(twice)
    assert rep.startswith("FAILED") and "reduced twice" in rep, rep
    missing = GOOD_ALLREDUCE.replace("1 0 reduce 1:out:0 0:in:0 16\n", "")
    rep = verify(missing)
    assert rep.startswith("FAILED") and "holds 1 contributions, expected 2" in rep, rep
    wrong_place = """
ranks 2 op allgather count 2
0 0 copy 0:out:0 0:in:0 8
0 0 copy 0:out:8 1:in:0 8
1 0 copy 1:out:0 1:in:0 8
1 0 copy 1:out:8 0:in:0 8
"""
    rep = verify(wrong_place)
    assert rep.startswith("FAILED") and "rank 1 output element 0" in rep, rep


def test_queues_of_one_rank_are_ordered_by_issue_order():
    # the second queue's task follows the first queue's in the issuing thread: no conflict between them
    two_queues = GOOD_ALLREDUCE.replace("0 0 reduce 0:out:0 1:in:0 16", "0 1 reduce 0:out:0 1:in:0 16")
    assert verify(two_queues).startswith("OK"), verify(two_queues)
