"""tf_rowstats_static (library-owned scratch) against tf_rowstats, through the exported C symbol.

Collected last on purpose: it must pass alone and after every other GPU test has used the device.
"""
import ctypes

import pytest
import torch

from titanic_flash_41_b200.ops import native

pytestmark = pytest.mark.gpu


def _static(lg, V, rows, temp, top_p, out, status):
    fn = native.lib().tf_rowstats_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return fn(lg.data_ptr() if lg is not None else None, V, V, rows, temp, top_p, out.data_ptr(),
              status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_rowstats_twice_in_a_row():
    dev = "cuda:0"
    sb = native.lib().tf_rowstat_bytes()
    st = native.StatusWord(dev)
    g = torch.Generator(device=dev).manual_seed(11)
    for call, (rows, V, temp, top_p) in enumerate(((5, 8192, 0.8, 0.9), (16, 4096 + 64, 1.3, 1.0))):
        lg = (torch.randn(rows, V, device=dev, generator=g) * 3).contiguous()
        want = torch.zeros(rows * sb, dtype=torch.uint8, device=dev)
        scr = torch.zeros(native.lib().tf_rowstats_scratch_bytes(rows), dtype=torch.uint8, device=dev)
        native.call("tf_rowstats", lg, V, V, rows, temp, top_p, want, scr, st.t)
        for rep in range(2):                                  # back to back on one stream
            got = torch.full((rows * sb,), 0xAB, dtype=torch.uint8, device=dev)
            assert _static(lg, V, rows, temp, top_p, got, st.t) == 0
            torch.cuda.synchronize()
            assert torch.equal(got, want), (call, rep)
    st.check()


def test_static_scratch_refuses_too_many_rows():
    dev = "cuda:0"
    st = native.StatusWord(dev)
    sb = native.lib().tf_rowstat_bytes()
    lg = torch.zeros(17, 1024, device=dev)
    out = torch.zeros(17 * sb, dtype=torch.uint8, device=dev)
    assert _static(lg, 1024, 17, 1.0, 1.0, out, st.t) == -3
    torch.cuda.synchronize()
    assert int(out.sum()) == 0                                 # nothing ran


def test_static_scratch_refuses_bad_arguments_on_the_host():
    """A bad argument is answered with -1 before anything is enqueued: no launch ever sees a null or
    short logits row, and a nucleus mass outside (0, 1] never reaches the kernels."""
    dev = "cuda:0"
    st = native.StatusWord(dev)
    sb = native.lib().tf_rowstat_bytes()
    rows, V = 4, 1024
    lg = torch.randn(rows, V, device=dev)
    out = torch.full((rows * sb,), 0xCD, dtype=torch.uint8, device=dev)
    fn = native.lib().tf_rowstats_static
    stream = torch.cuda.current_stream().cuda_stream
    assert _static(None, V, rows, 1.0, 1.0, out, st.t) == -1                     # null logits
    assert fn(lg.data_ptr(), V - 4, V, rows, 1.0, 1.0, out.data_ptr(), st.t.data_ptr(), stream) == -1   # ldl < V
    assert _static(lg, V, rows, 1.0, 0.0, out, st.t) == -1                      # top_p = 0
    assert _static(lg, V, rows, 1.0, float("nan"), out, st.t) == -1
    assert _static(lg, V, rows, 0.0, 1.0, out, st.t) == -1                      # temperature = 0
    torch.cuda.synchronize()
    assert (out == 0xCD).all()                                 # untouched
    st.check()
