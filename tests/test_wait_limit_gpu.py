"""A device-side wait that runs out: the kernel gives up by itself, the host reads an error status, a reset
restores service.  The waits are made to run out by giving them a short poll limit (``b200_set_wait_limit``) and
a peer that never answers (a second buffer on the same GPU whose flags nobody raises): nothing faults, nothing
hangs, no process dies."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

KEY_FLAGS, KEY_COUNT, KEY_ERR, KEYS, FLAG_STRIDE = 1024, 1536, 1540, 2048, 64      # csrc/tp_layout.cuh


@pytest.fixture()
def short_waits(be, cuda):
    lib = be._lib.lib()
    lib.b200_set_wait_limit(4096)
    yield lib
    lib.b200_set_wait_limit(0)


def _buffers(lib, cuda, hidden):
    nbytes = lib.b200_forward_tp_buffer_bytes(hidden)
    own = torch.zeros(nbytes, dtype=torch.uint8, device=cuda)
    peer = torch.zeros(nbytes, dtype=torch.uint8, device=cuda)
    arr = (ctypes.c_void_p * 8)(own.data_ptr(), peer.data_ptr())
    return nbytes, own, peer, arr


def test_argmax_combine_gives_up_reports_and_recovers(be, cuda, short_waits):
    lib, p = short_waits, be._lib.ptr
    nbytes, own, peer, arr = _buffers(lib, cuda, 256)
    st = be._lib.stream_ptr(cuda)
    mine = (torch.arange(1, 9, dtype=torch.int64, device=cuda) << 32) | 0xFFFFFF00
    keys = mine.clone()
    assert lib.b200_tp_argmax_combine(p(keys), 8, 0, 2, 0, arr, st) == 0
    torch.cuda.synchronize()                                     # returns: the wait ran out after 4096 polls
    assert lib.b200_tp_exchange_error(ctypes.c_void_p(own.data_ptr())) == 1
    assert torch.equal(keys, mine)                               # nothing was combined
    # the host's recovery: zero the buffers, then a combine whose peer does answer (the test plays the peer:
    # its keys in its buffer, its flag in ours) succeeds and the error word stays clear
    assert lib.b200_tp_exchange_reset(ctypes.c_void_p(own.data_ptr()), nbytes) == 0
    assert lib.b200_tp_exchange_reset(ctypes.c_void_p(peer.data_ptr()), nbytes) == 0
    theirs = (torch.tensor([9, 1, 9, 1, 9, 1, 9, 1], dtype=torch.int64, device=cuda) << 32) | 0xFFFFFF00
    peer[KEYS:KEYS + 64].view(torch.int64).copy_(theirs)
    own[KEY_FLAGS + FLAG_STRIDE:KEY_FLAGS + FLAG_STRIDE + 4].view(torch.int32).fill_(1)
    keys = mine.clone()
    assert lib.b200_tp_argmax_combine(p(keys), 8, 0, 2, 0, arr, st) == 0
    torch.cuda.synchronize()
    assert lib.b200_tp_exchange_error(ctypes.c_void_p(own.data_ptr())) == 0
    assert torch.equal(keys, torch.maximum(mine, theirs))
    assert int(own[KEY_COUNT:KEY_COUNT + 4].view(torch.int32)) == 1


def test_forward_all_gpu_barrier_gives_up_and_the_model_recovers(be, cuda, short_waits):
    lib = short_waits
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device=cuda, gen_device="cpu")
    prompt = torch.arange(5, 17, dtype=torch.int32)
    whole = be.Model.random_init(args, seed=11, device=cuda, gen_device="cpu").relayout()
    want = whole(prompt[None], cache=whole.make_cache(128))
    shard = base.shard(0, 2).relayout()
    nbytes, own, peer, arr = _buffers(lib, cuda, args.hidden_size)
    shard.tp.peers, shard.tp.peer_array, shard.tp.nbytes = [own.data_ptr(), peer.data_ptr()], arr, nbytes
    assert shard.can_fuse()
    shard(prompt[None], cache=shard.make_cache(128))             # rank 1 does not exist: its arrivals never come
    torch.cuda.synchronize()                                     # ... and the kernel still ends
    with pytest.raises(be._lib.B200Error, match="code 12"):
        shard.check_fused_error()                                # also clears the kernel's barrier words
    assert lib.b200_tp_exchange_reset(ctypes.c_void_p(own.data_ptr()), nbytes) == 0
    # the GPU and the library stay usable: the unsharded model gives its usual logits
    again = whole(prompt[None], cache=whole.make_cache(128))
    whole.check_fused_error()
    assert torch.equal(again, want)
