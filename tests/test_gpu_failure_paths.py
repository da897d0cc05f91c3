"""Failure paths that can be exercised without faulting, trapping or hanging a GPU.

Every wait inside this library's kernels is bounded and reports through a host-visible word. The
only one that can be made to run out on purpose and cheaply is the arrival wait of the
tensor-parallel exchange: a two-rank exchange on ONE device whose "peer" region is a second local
allocation whose flag nobody raises, with the wait limited to a few thousand polls (about a
millisecond). The kernel must give up, say which rank was missing, finish, and leave the device
usable.
"""
import ctypes as C

import numpy as np
import pytest

from dyninfer_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_exchange_wait_runs_out_and_is_reported(native_lib):
    rc = native_lib.dyninfer_cuda_tp_exchange_wait_probe(1024, 3, 4000)
    assert rc != 0
    msg = _lib.last_error()
    assert "rank 1 did not arrive within the wait limit" in msg and "rank 0 gave up" in msg
    # the context is intact: an ordinary product still runs and is right
    w = synth.random_weight("gguf.q4_0", 64, 256, 9)["data"]
    dw = ops.DeviceWeight("gguf.q4_0", 64, 256, w)
    x = torch.ones(1, 256, device="cuda")
    y = ops.linear(dw, x).cpu().numpy()
    assert np.isfinite(y).all()
    ops.check_device_error()
    # argument checks of the probe itself
    assert native_lib.dyninfer_cuda_tp_exchange_wait_probe(1023, 3, 4000) != 0
    assert native_lib.dyninfer_cuda_tp_exchange_wait_probe(1024, 3, 0) != 0


def test_device_error_word_starts_clear(native_lib):
    assert native_lib.dyninfer_cuda_check_device_error() == 0


def test_page_and_chunk_sizes_must_divide(native_lib, tmp_path):
    """wrapper.c:921: neither size divides the other -> invalid configuration."""
    from dyninfer_b200 import DynInferError
    from dyninfer_b200.runtime import ModelLoader
    path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), synth.TINY, seed=2)
    model = ModelLoader().load(path, max_kv=512, chunk_size=96)      # pages are 256 tokens
    with pytest.raises(DynInferError, match="do not divide one another"):
        model.create_session()
