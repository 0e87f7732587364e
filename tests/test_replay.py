"""Recording launcher calls and issuing them again from native code, on the host: the generic call passes every
argument where the launcher expects it (registers, stack slots, float registers), pointers are swapped only
where they are marked as pointers, and a launcher's refusal comes back with its message (no GPU needed)."""
import ctypes

import pytest

from microllm_rocm_b200.kernels import ops, replay
from microllm_rocm_b200.kernels.build import KernelError


def probe_args(out, p0=0x1000, p3=0x2000, a2=7):
    return (p0, -5_000_000_000, a2, 1.5, p3, 11, -12, 13, 1 << 40, -0.25, 99, ctypes.addressof(out))


def test_recorded_calls_come_back_with_every_argument_in_place():
    L = ops.lib("replay.cu")
    out = (ctypes.c_longlong * 11)()
    with replay.Recorder() as rec:
        assert L.mlb_replay_probe(*probe_args(out)) == 0
        assert L.mlb_replay_probe(*probe_args(out, p0=0x3000, a2=8)) == 0
    direct = list(out)
    assert direct == [0x3000, -5_000_000_000, 8, 0x2000, 11, -12, 13, 1 << 40, 99, 1500, -250]
    recording = replay.Recording(rec)
    assert recording.count == 2 and {0x1000, 0x2000, 0x3000, ctypes.addressof(out)} <= recording.pointers
    for i in range(11):
        out[i] = 0
    assert recording.replay([]) == 2
    assert list(out) == direct                       # the second call wrote last
    # swap 0x3000 and 0x2000 for other addresses; the integer 13 and the long long 1 << 40 are no pointers and stay
    for i in range(11):
        out[i] = 0
    recording.replay([(0x3000, 0x7000), (0x2000, 0x8000), (13, 555), (1 << 40, 1)])
    assert list(out) == [0x7000, -5_000_000_000, 8, 0x8000, 11, -12, 13, 1 << 40, 99, 1500, -250]


def test_a_refusing_launcher_ends_the_replay_with_its_message():
    L = ops.lib("replay.cu")
    out = (ctypes.c_longlong * 11)()
    with replay.Recorder() as rec:
        L.mlb_replay_probe(*probe_args(out, a2=-3))          # refuses, and is recorded all the same
        L.mlb_replay_probe(*probe_args(out, a2=4))
    recording = replay.Recording(rec)
    with pytest.raises(KernelError, match="refused on purpose"):
        recording.replay([])
    assert out[2] == -3                                      # the call after the refusal was not made


def test_nothing_is_recorded_without_a_recorder():
    L = ops.lib("replay.cu")
    out = (ctypes.c_longlong * 11)()
    assert L.mlb_replay_probe(*probe_args(out)) == 0
    with replay.Recorder() as rec:
        pass
    assert rec.calls == [] and replay._active is None
