"""The peer exchange when a peer never arrives, on ONE GPU and without a fault: a world-2
context whose second rank is a block of memory the test owns.  Nothing ever stores rank 1's
partial sums, so the reader's bounded wait runs out: the kernel returns by itself, the device
status word reads AB2_ERR_TIMEOUT, the context stays usable.  After ab2_tp_peer_reset the test
plays the missing peer itself (it writes rank 1's words {sum, exchange number} into rank 0's
inbox) and the exchange gives the right sums again."""
import numpy as np
import pytest
import torch

from helpers import pkg

pytestmark = pytest.mark.gpu


def _ll_words(values, exchange):
    """{f32 sum, u32 exchange number} as 8-byte words."""
    v = np.ascontiguousarray(values, np.float32).view(np.uint32).astype(np.uint64)
    return torch.from_numpy((v | (np.uint64(exchange) << np.uint64(32))).view(np.int64))


def test_wait_runs_out_then_reset_restores_the_exchange():
    p = pkg()
    n, max_elems, world = 4096, 4096, 2
    tp = p.TensorParallel(0, world, None)              # no communicator: the peer exchange only
    block, nbytes = tp.export_block(max_elems)
    fake_peer = torch.zeros(nbytes // 8, dtype=torch.int64, device="cuda")   # rank 1's inbox: nobody reads it
    tp.attach_blocks([block, fake_peer.data_ptr()])
    tp.set_wait_limit_ns(5_000_000)                    # 5 ms
    mine = torch.arange(n, dtype=torch.float32, device="cuda") * 0.25
    x0 = torch.ones(n, dtype=torch.bfloat16, device="cuda")

    # 1. rank 1 never deposits: the wait runs out, the status word says so, nothing hangs
    x = x0.clone()
    tp.peer_deposit(mine)
    tp.peer_reduce_add(x)
    assert p.device_status() == -6
    assert p.device_status() == 0                      # reading the word clears it

    # 2. reset, then the test plays rank 1: exchange 1 uses buffer 1, rank r's slot is [buffer][r]
    tp.peer_reset()
    theirs = np.linspace(-3.0, 5.0, n).astype(np.float32)
    slot = (1 * world + 1) * max_elems                 # buffer 1, rank 1
    _copy_into(block + slot * 8, _ll_words(theirs, 1).cuda())
    x = x0.clone()
    tp.peer_deposit(mine)
    tp.peer_reduce_add(x)
    assert p.device_status() == 0
    want = (x0.float() + (mine + torch.from_numpy(theirs).cuda()).to(torch.bfloat16).float()).to(torch.bfloat16)
    assert torch.equal(x, want)

    # 3. the next exchange (number 2, buffer 0) works the same way
    _copy_into(block + (0 * world + 1) * max_elems * 8, _ll_words(theirs * 2, 2).cuda())
    x = x0.clone()
    tp.peer_deposit(mine)
    tp.peer_reduce_add(x)
    assert p.device_status() == 0
    want = (x0.float() + (mine + 2 * torch.from_numpy(theirs).cuda()).to(torch.bfloat16).float()).to(torch.bfloat16)
    assert torch.equal(x, want)


def _copy_into(dev_ptr, src: torch.Tensor):
    """Device-to-device copy of a tensor to a raw device address."""
    import ctypes as C
    rt = None
    for name in ("libcudart.so.12", "libcudart.so"):
        try:
            rt = C.CDLL(name)
            break
        except OSError:
            continue
    assert rt is not None, "CUDA runtime library not found"
    rc = rt.cudaMemcpy(C.c_void_p(dev_ptr), C.c_void_p(src.data_ptr()), C.c_size_t(src.numel() * src.element_size()), 3)
    assert rc == 0
    torch.cuda.synchronize()
