"""LayerNorm backward through the entry point that takes no workspace.

Some hosts of this library cannot give a kernel scratch memory when they call
it (they sit inside a stream capture, or their pool was sized once at start-up
and may not grow), so mograd_b200_layer_norm_bwd_static keeps its scratch in a
fixed array inside the library.  This file checks, through the C ABI, that it
returns exactly what the workspace-taking entry point returns, twice in a row
with different shapes (the second call sees the first call's leftovers in the
shared array), and that it refuses sizes the array cannot hold.  It is named
to be collected last so that a fail-fast run has already run everything else.
"""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


def _run_both(cuda, rows, cols, dtype, seed):
    import torch
    from mograd_b200 import _lib
    from mograd_b200 import dispatch as K

    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((rows, cols), generator=g).to(cuda).to(dtype)
    dy = torch.randn((rows, cols), generator=g).to(cuda).to(dtype)
    gamma = (1 + 0.1 * torch.randn(cols, generator=g)).to(cuda).to(dtype)
    want = K.layer_norm_bwd_dispatch(dy, x, gamma)
    dx, dg, db = torch.full_like(x, float("nan")), torch.full_like(gamma, float("nan")), torch.full_like(gamma, float("nan"))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.call("mograd_b200_layer_norm_bwd_static", p(dy), p(x), p(gamma), p(dx), p(dg), p(db), rows, cols, 1e-5,
              K.dtype_code(x), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return want, (dx, dg, db)


def test_static_scratch_matches_workspace_entry_point_twice(cuda):
    import torch

    # same kernels, same launch plan: the results must be identical, not merely close
    # (64, 8192): rows wider than 4096 are accepted while the launch is small enough for the array
    for rows, cols, dtype, seed in ((4099, 768, torch.bfloat16, 0), (513, 4096, torch.float32, 1),
                                    (4099, 768, torch.bfloat16, 2), (64, 8192, torch.bfloat16, 3)):
        want, got = _run_both(cuda, rows, cols, dtype, seed)
        for w, g in zip(want, got):
            assert torch.isfinite(g.float()).all()
            assert torch.equal(w, g)


def test_static_scratch_rejects_what_does_not_fit(cuda):
    import torch
    from mograd_b200 import _lib

    x = torch.zeros((4096, 16384), device=cuda)
    gamma = torch.ones(16384, device=cuda)
    out = torch.empty_like(x)
    dg, db = torch.empty_like(gamma), torch.empty_like(gamma)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    with pytest.raises(_lib.KernelError) as e:
        _lib.call("mograd_b200_layer_norm_bwd_static", p(x), p(x), p(gamma), p(out), p(dg), p(db), 4096, 16384, 1e-5,
                  _lib.F32, None)
    assert e.value.code == _lib.EUNSUPPORTED and "built-in array" in e.value.message
