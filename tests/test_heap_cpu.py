"""Host-side parts of the symmetric arena: the free list, and the file-descriptor exchange between ranks
(run as three gloo processes on CPU; the descriptors here are memory files instead of GPU memory handles)."""
import os

import pytest

from test_dist_cpu import run_ranks


def test_free_list_first_fit_and_coalescing():
    from mgwfbp_b200.parallel.comm.heap import FreeList
    fl = FreeList(4096)
    a = fl.take(100)          # rounded to 256
    b = fl.take(300)          # rounded to 512
    c = fl.take(256)
    assert (a, b, c) == (0, 256, 768)
    assert fl.used() == 1024
    fl.give(b, 300)
    assert fl.take(600) == 1024           # the 512-byte hole is too small
    assert fl.take(512) == 256            # ... but fits this one exactly
    fl.give(a, 100)
    fl.give(256, 512)
    fl.give(c, 256)
    assert fl.free[0] == (0, 1024)        # three neighbours merged into one block
    fl.give(1024, 600)
    assert fl.free == [(0, 4096)]
    assert fl.take(8192) is None
    with pytest.raises(ValueError):
        fl.give(0, 256)                   # already free


def _swap_pipes(rank, world):
    from mgwfbp_b200.parallel.comm.heap import exchange_fds
    r = os.memfd_create('mgw-test')               # every receiver reads the same bytes (a pipe would be drained by the first)
    os.write(r, b'hello from %d' % rank)
    got = exchange_fds(r, list(range(world)))
    os.close(r)
    texts = {}
    for sender, fd in got.items():
        texts[sender] = os.pread(fd, 64, 0).decode()
        os.close(fd)
    # a second round with a single sender, the way the multicast handle travels
    r2 = os.memfd_create('mgw-test-root')
    os.write(r2, b'root')
    got2 = exchange_fds(r2 if rank == 0 else None, [0])
    os.close(r2)
    root = None
    for sender, fd in got2.items():
        root = (sender, os.pread(fd, 16, 0).decode())
        os.close(fd)
    return texts, root


def test_descriptor_exchange_between_processes():
    res = run_ranks(_swap_pipes, (), world=3)
    for rank, (texts, root) in enumerate(res):
        assert texts == {s: 'hello from %d' % s for s in range(3) if s != rank}
        assert root == (None if rank == 0 else (0, 'root'))
