"""The launch recorder of ``kernels.py`` on the CPU, with the C library standing in for the kernel
library: a recorded list repeats the calls with the same arguments; query functions are not
wrapped; a signature declared on what the wrapper hands out lands on the ctypes function itself."""
import ctypes

import pytest

from aien_sovereign_core_mv_b200 import kernels as K


@pytest.fixture()
def libc():
    return K._Library(ctypes.CDLL(None))


def test_signature_declared_on_the_wrapper_reaches_the_function(libc):
    f = libc.labs
    f.argtypes = [ctypes.c_long]
    f.restype = ctypes.c_long
    raw = libc._cdll.labs
    assert raw.argtypes == [ctypes.c_long] and raw.restype is ctypes.c_long
    assert f(-(1 << 40)) == 1 << 40               # a 64-bit argument survives: the declaration is in force
    assert libc.labs is f                          # looked up once


def test_recorded_calls_are_issued_again():
    calls = []
    proto = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int, ctypes.c_int)

    def launch(a, b):
        calls.append((a, b))
        return 0
    fn = proto(launch)
    entry = K._Entry(fn)
    entry(1, 2)                                    # not recording
    K.begin_recording()
    entry(3, 4)
    entry(5, 6)
    plan = K.end_recording()
    assert [args for _, args in plan] == [(3, 4), (5, 6)]
    before = K.launch_count()
    K.replay_launches(plan)
    assert calls == [(1, 2), (3, 4), (5, 6), (3, 4), (5, 6)]
    assert K.launch_count() == before + 2
    entry(7, 8)                                    # recording has ended
    assert len(plan) == 2


def test_a_failing_call_in_a_replay_raises():
    proto = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int)
    fn = proto(lambda code: code)
    with pytest.raises(K.KernelError):
        K.replay_launches([(fn, (-3,))])


def test_query_functions_are_not_wrapped(libc):
    class Fake:
        def __init__(self):
            self.aien_thing_supports = lambda *a: 1
            self.aien_thing = lambda *a: 0
    lib = K._Library(Fake())
    assert not isinstance(lib.aien_thing_supports, K._Entry)
    assert isinstance(lib.aien_thing, K._Entry)
