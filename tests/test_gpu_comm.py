"""The peer-memory exchange kernel (``bxl_comm_exchange``) on ONE GPU.  The peers are not
running: their buffers and control words are ordinary tensors on the same device, and what they
would have signalled is written into this rank's control words beforehand, so the kernel never
waits on another launch.  Checked: the contribution lands in every peer's buffer, the sequence
number is published to every peer, the ticket is reset, consecutive calls advance the sequence,
and a wait that nobody answers gives up within its limit and is reported through the device
status word (the context stays usable)."""
import ctypes as C

import pytest
import torch

from tests._util import cuda_or_skip

pytestmark = pytest.mark.gpu
SENT, READY, SEQ, TICKET = 0, 8, 16, 17  # control-word layout (include/basedxl_b200.h: bxl_comm_exchange)


def _exchange(l, _lib, src, dsts, ctl, peer_ctls, own, handshake=False, wait=0.25):
    n = len(dsts)
    vp = C.c_void_p
    dst = (vp * n)(*[(None if d is None else d.data_ptr()) for d in dsts])
    pc = (vp * n)(*[(None if c is None else c.data_ptr()) for c in peer_ctls])
    _lib.check(l.bxl_comm_exchange(src.data_ptr(), dst, src.numel() * src.element_size(), ctl.data_ptr(), pc, n, own, int(handshake),
                                   float(wait), torch.cuda.current_stream().cuda_stream), l)


@pytest.mark.parametrize("n,own", [(2, 0), (4, 1), (8, 7)])
@pytest.mark.parametrize("numel", [8, 4096 + 8, 1 << 20])
def test_exchange_delivers_and_signals(n, own, numel):
    dev = cuda_or_skip()
    from basedxl_b200 import _lib

    l = _lib.lib()
    words = l.bxl_comm_ctl_bytes() // 4
    g = torch.Generator(device="cuda").manual_seed(n + numel)
    ctl = torch.zeros(words, dtype=torch.int32, device=dev)
    peer_ctl = [None if p == own else torch.zeros(words, dtype=torch.int32, device=dev) for p in range(n)]
    dsts = [None if p == own else torch.zeros(numel, dtype=torch.float16, device=dev) for p in range(n)]
    # the peers' arrivals for the next 1000 exchanges are already on record
    ctl[SENT : SENT + n] = 1000
    ctl[READY : READY + n] = 1000
    for call in (1, 2, 3):
        src = torch.randn(numel, device=dev, generator=g).half()
        _exchange(l, _lib, src, dsts, ctl, peer_ctl, own, handshake=(call == 3))
        _lib.device_status()
        for p in range(n):
            if p == own:
                continue
            assert torch.equal(dsts[p], src), f"peer {p} did not receive the contribution of call {call}"
            assert int(peer_ctl[p][SENT + own]) == call, "sequence number not published to the peer"
            assert int(peer_ctl[p][READY + own]) == (3 if call == 3 else 0)
        assert int(ctl[SEQ]) == call and int(ctl[TICKET]) == 0


def test_unanswered_wait_times_out_and_is_reported():
    dev = cuda_or_skip()
    from basedxl_b200 import _lib

    l = _lib.lib()
    words = l.bxl_comm_ctl_bytes() // 4
    ctl = torch.zeros(words, dtype=torch.int32, device=dev)
    peer_ctl = [None, torch.zeros(words, dtype=torch.int32, device=dev)]
    dst = torch.zeros(64, dtype=torch.float16, device=dev)
    src = torch.ones(64, dtype=torch.float16, device=dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    _exchange(l, _lib, src, [None, dst], ctl, peer_ctl, 0, wait=0.2)   # the peer never signals
    t1.record()
    with pytest.raises(_lib.BxlError, match="wait site 901"):
        _lib.device_status()
    assert 150.0 < t0.elapsed_time(t1) < 2000.0
    # the data had been delivered before the wait; the library and the context remain usable
    assert torch.equal(dst, src)
    _lib.device_status()
    ctl[SENT + 1] = 1000
    _exchange(l, _lib, src * 2, [None, dst], ctl, peer_ctl, 0)
    _lib.device_status()
    assert torch.equal(dst, src * 2)


def test_bad_arguments_are_rejected():
    dev = cuda_or_skip()
    from basedxl_b200 import _lib

    l = _lib.lib()
    words = l.bxl_comm_ctl_bytes() // 4
    ctl = torch.zeros(words, dtype=torch.int32, device=dev)
    src = torch.ones(64, dtype=torch.float16, device=dev)
    with pytest.raises(_lib.BxlError):
        _exchange(l, _lib, src, [None] * 9, ctl, [None] * 9, 0)          # more peers than supported
    with pytest.raises(_lib.BxlError):
        _exchange(l, _lib, src, [None, src], ctl, [None, None], 0)       # a peer without control words
    with pytest.raises(_lib.BxlError):
        _exchange(l, _lib, src[:4], [None, src[:4]], ctl, [None, ctl], 0)  # 8 bytes: not a whole 16-byte vector
