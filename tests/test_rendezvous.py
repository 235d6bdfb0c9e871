"""The host-side rendezvous of a GPU pair (flux_cuda_rendezvous_*), exercised between CPU threads standing in for the
two GPUs' host threads: what a member sees when its partner is on time, late, missing, or has given up. No GPU is
involved, so the failure cases cost nothing but the timeout they test."""
import ctypes
import threading
import time

OK, PEER_TIMEOUT = 0, -7


def _make(fx, parties=2):
    h = ctypes.c_void_p()
    assert fx.lib().flux_cuda_rendezvous_create(parties, ctypes.byref(h)) == 0
    return h


def test_both_members_arrive(fx):
    L = fx.lib()
    r = _make(fx)
    got = {}

    def member(rank, delay):
        for step in range(1, 6):
            time.sleep(delay)
            got[(rank, step)] = L.flux_cuda_rendezvous_arrive_and_wait(r, rank, step, 5000)

    th = [threading.Thread(target=member, args=(0, 0.0)), threading.Thread(target=member, args=(1, 0.02))]
    [t.start() for t in th]
    [t.join() for t in th]
    assert all(v == OK for v in got.values()) and len(got) == 10
    L.flux_cuda_rendezvous_destroy(r)


def test_a_member_that_never_arrives_times_the_other_out(fx):
    L = fx.lib()
    r = _make(fx)
    t0 = time.perf_counter()
    rc = L.flux_cuda_rendezvous_arrive_and_wait(r, 0, 1, 150)
    dt = time.perf_counter() - t0
    assert rc == PEER_TIMEOUT and 0.14 <= dt < 2.0
    assert b"did not reach step 1" in L.flux_cuda_last_error()
    # the late member finds its partner already there and goes through; the next step times out again
    assert L.flux_cuda_rendezvous_arrive_and_wait(r, 1, 1, 150) == OK
    assert L.flux_cuda_rendezvous_arrive_and_wait(r, 1, 2, 50) == PEER_TIMEOUT
    L.flux_cuda_rendezvous_destroy(r)


def test_a_member_that_gives_up_releases_the_other_at_once(fx):
    L = fx.lib()
    r = _make(fx)
    out = {}

    def waiter():
        t0 = time.perf_counter()
        out["rc"] = L.flux_cuda_rendezvous_arrive_and_wait(r, 0, 3, 10000)
        out["dt"] = time.perf_counter() - t0
        out["msg"] = L.flux_cuda_last_error()  # the error text is per thread: read it where it was set

    t = threading.Thread(target=waiter)
    t.start()
    time.sleep(0.1)
    L.flux_cuda_rendezvous_abandon(r, 1)  # member 1's forward pass failed: it will not come
    t.join()
    assert out["rc"] == PEER_TIMEOUT and out["dt"] < 2.0
    assert b"gave up" in out["msg"]
    L.flux_cuda_rendezvous_destroy(r)


def test_arguments_are_checked(fx):
    L = fx.lib()
    h = ctypes.c_void_p()
    assert L.flux_cuda_rendezvous_create(0, ctypes.byref(h)) != 0
    r = _make(fx)
    assert L.flux_cuda_rendezvous_arrive_and_wait(r, 2, 1, 10) != 0
    assert L.flux_cuda_rendezvous_arrive_and_wait(r, 0, 1, -1) != 0
    L.flux_cuda_rendezvous_destroy(r)
    # without a GPU the group itself cannot exist, and says so
    import torch
    if not torch.cuda.is_available():
        g = ctypes.c_void_p()
        assert L.flux_cuda_group_create(2, None, ctypes.byref(g)) != 0 and not g.value
