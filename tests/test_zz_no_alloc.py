"""The allocation-free lm_head log-prob entry point, called through its exported C symbol, must agree with the
existing entry point (which takes caller-provided scratch) on consecutive calls that reuse the built-in scratch."""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from verl_b200.ops import _ext

    _ext.load()
    import verl_b200

    path = os.path.join(os.path.dirname(verl_b200.__file__), "_C.so")
    lib = ctypes.CDLL(path)
    vp, i, f, l = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long
    lib.vb_lmhead_scratch_floats.restype = l
    lib.vb_lmhead_scratch_floats.argtypes = [i, i]
    lib.vb_lmhead_static_capacity_floats.restype = l
    lib.vb_lmhead_static_capacity_floats.argtypes = []
    lib.vb_lmhead_logprob_fwd.restype = i
    lib.vb_lmhead_logprob_fwd.argtypes = [vp, vp, vp, i, i, i, i, i, f, vp, vp, vp, vp, vp, vp]
    lib.vb_lmhead_logprob_fwd_static.restype = i
    lib.vb_lmhead_logprob_fwd_static.argtypes = [vp, vp, vp, i, i, i, i, i, f, vp, vp, vp, vp, vp]
    return lib


def _case(M, V, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    h = (0.5 * torch.randn(M, K, device="cuda", generator=g)).bfloat16()
    w = (0.05 * torch.randn(V, K, device="cuda", generator=g)).bfloat16()
    labels = torch.randint(0, V, (M,), device="cuda", generator=g)
    return h, w, labels


def _run_both(lib, h, w, labels, inv_temp, with_ent=True, with_lse=True):
    M, K = h.shape
    V = w.shape[0]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    for static in (False, True):
        logp, ent, lse = (torch.full((M,), float("nan"), device="cuda") for _ in range(3))
        common = (h.data_ptr(), w.data_ptr(), labels.data_ptr(), M, V, K, h.stride(0), w.stride(0), inv_temp)
        tail = (logp.data_ptr(), ent.data_ptr() if with_ent else None, lse.data_ptr() if with_lse else None, err.data_ptr(), stream)
        if static:
            rc = lib.vb_lmhead_logprob_fwd_static(*common, *tail)
        else:
            scratch = torch.empty(lib.vb_lmhead_scratch_floats(M, V), device="cuda")
            rc = lib.vb_lmhead_logprob_fwd(*common, scratch.data_ptr(), *tail)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        outs.append((logp, ent, lse))
    return outs


def test_static_scratch_entry_point_matches_on_two_calls_in_a_row():
    lib = _lib()
    # second call is smaller and uses other data, so anything left in the shared scratch by the first would show
    for M, V, K, seed, inv_temp in ((1000, 5000, 512, 1, 1.0), (333, 2100, 256, 2, 0.7)):
        assert lib.vb_lmhead_scratch_floats(M, V) <= lib.vb_lmhead_static_capacity_floats()
        h, w, labels = _case(M, V, K, seed)
        (lp0, en0, ls0), (lp1, en1, ls1) = _run_both(lib, h, w, labels, inv_temp)
        torch.testing.assert_close(lp1, lp0, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(en1, en0, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(ls1, ls0, rtol=1e-5, atol=1e-5)
        logits = (h.float() @ w.float().t()) * inv_temp
        ref = torch.log_softmax(logits, -1).gather(1, labels[:, None])[:, 0]
        torch.testing.assert_close(lp1, ref, rtol=2e-2, atol=2e-2)


def test_labels_outside_the_vocabulary_and_optional_outputs():
    """Rows whose label is not a column of W (ignore index, padded vocabulary) must give logp = -lse in BOTH entry points,
    also when the shared scratch still holds the label logits of an earlier, larger call; ent / lse may be left out."""
    lib = _lib()
    h, w, labels = _case(900, 4000, 256, 7)
    _run_both(lib, h, w, labels, 1.0)                       # fills the built-in scratch with in-range label logits
    M, V, K = 300, 2100, 256
    h, w, labels = _case(M, V, K, 8)
    labels[::7] = -100
    labels[3::11] = V + 5
    bad = (labels < 0) | (labels >= V)
    assert int(bad.sum()) > 20
    (lp0, en0, ls0), (lp1, en1, ls1) = _run_both(lib, h, w, labels, 1.0)
    torch.testing.assert_close(lp1, lp0, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lp1[bad], -ls1[bad], rtol=0, atol=0)
    torch.testing.assert_close(lp0[bad], -ls0[bad], rtol=0, atol=0)
    # without the optional outputs the log-probs are unchanged and the skipped buffers stay untouched (NaN-filled)
    (lpa, ena, lsa), (lpb, enb, lsb) = _run_both(lib, h, w, labels, 1.0, with_ent=False, with_lse=False)
    torch.testing.assert_close(lpb, lp1, rtol=0, atol=0)
    torch.testing.assert_close(lpa, lp0, rtol=0, atol=0)
    assert bool(torch.isnan(enb).all()) and bool(torch.isnan(lsb).all())


def test_static_scratch_entry_point_rejects_sizes_beyond_its_capacity():
    lib = _lib()
    M, V, K = 8192, 152064, 64
    assert lib.vb_lmhead_scratch_floats(M, V) > lib.vb_lmhead_static_capacity_floats()
    # rejected on the host before anything is launched; the pointers are never touched
    h = torch.zeros(8, K, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8, device="cuda")
    rc = lib.vb_lmhead_logprob_fwd_static(h.data_ptr(), h.data_ptr(), out.data_ptr(), M, V, K, K, K, 1.0, out.data_ptr(), None, None,
                                          out.data_ptr(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -20
