"""The allocation-free SSD entry point (qb_ssd_chunk_scan_fwd_noalloc).

It exists for callers that cannot give the library scratch memory -- a host program with no device
allocator of its own, or one whose pool is sealed after model load -- so the workspace comes from an
array inside the library.  The test calls it through the C ABI twice in a row (the array keeps the
first call's contents, the second call must not be disturbed by them) and requires the outputs of
both calls to equal those of the regular entry point, which gets a fresh caller-owned workspace.
The file name makes pytest collect it last."""
import ctypes

import pytest
import torch

from helpers import make_ssd_case

pytestmark = pytest.mark.gpu


def _args(lib_mod, c, dev_t, out, fin, ws, ws_bytes, Bsz, L, H, P, G, N, Q):
    p = lambda t: None if t is None else t.data_ptr()
    return lib_mod.make(
        "qb_ssd_args", x=p(dev_t["q_x"]), dt=p(dev_t["q_dt"]), Bm=p(dev_t["q_B"]), Cm=p(dev_t["q_C"]), A_log=p(dev_t["q_A_log"]),
        D=p(dev_t["q_D"]), z=None, dt_bias=p(dev_t["dt_bias"]), x_scales=p(dev_t["x_scales"]), dt_scale=p(dev_t["s_dt"]),
        A_scale=p(dev_t["s_A"]), B_scale=p(dev_t["s_B"]), C_scale=p(dev_t["s_C"]), D_scale=p(dev_t["s_D"]), z_scale=None,
        ssm_state_scale=p(dev_t["state_scale"]), head_group_range=None, dim_group_range=None, out=p(out), final_states=p(fin),
        workspace=p(ws), workspace_bytes=ws_bytes, x_sb=L * H * P, x_sl=H * P, x_sh=P, dt_sb=L * H, dt_sl=H,
        B_sb=L * G * N, B_sl=G * N, B_sg=N, C_sb=L * G * N, C_sl=G * N, C_sg=N, batch=Bsz, seqlen=L, nheads=H, headdim=P,
        ngroups=G, dstate=N, chunk_size=Q, grouped=0, nhead_groups=0, ndim_groups=0, D_has_hdim=0, dt_softplus=1,
        dt_min=0.0, dt_max=3.0e38)


@pytest.mark.parametrize("portable", [False, True])
def test_noalloc_entry_point_matches_regular_one_twice(portable):
    """``portable`` sends both entry points down the five-stage path (cumulative sums, C B^T, chunk states, state
    passing, output), whose stages read back what earlier stages left in the scratch array; the default shapes take the
    single tensor-core kernel."""
    from quamba_b200 import _lib
    if portable:
        with _lib.path_override(_lib.PATH_SSD_PORTABLE):
            _twice(_lib)
    else:
        _twice(_lib)


def _twice(_lib):
    lib = _lib.lib()
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.qb_ssd_static_scratch_bytes() == 48 << 20
    for call, (L, seed) in enumerate([(600, 11), (333, 12)]):          # two calls in a row, different shapes and data
        Bsz, H, P, G, N, Q = 2, 8, 64, 1, 128, 256
        c = make_ssd_case(Bsz, L, H, P, G, N, Q, seed=seed)
        d = {k: (v.to(dev).contiguous() if torch.is_tensor(v) else v) for k, v in c.items()}
        ws_bytes = lib.qb_ssd_workspace_bytes(Bsz, L, H, P, G, N, Q)
        assert 0 < ws_bytes <= lib.qb_ssd_static_scratch_bytes()
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        out_a = torch.zeros(Bsz, L, H, P, dtype=torch.float16, device=dev)
        fin_a = torch.zeros(Bsz, H, P, N, dtype=torch.int8, device=dev)
        out_b, fin_b = torch.ones_like(out_a), torch.ones_like(fin_a)
        a = _args(_lib, c, d, out_a, fin_a, ws, ws_bytes, Bsz, L, H, P, G, N, Q)
        _lib.check(lib.qb_ssd_chunk_scan_fwd(ctypes.byref(a), ctypes.c_void_p(stream)))
        b = _args(_lib, c, d, out_b, fin_b, None, 0, Bsz, L, H, P, G, N, Q)     # no workspace from the caller
        _lib.check(lib.qb_ssd_chunk_scan_fwd_noalloc(ctypes.byref(b), ctypes.c_void_p(stream)))
        torch.cuda.synchronize()
        _lib.read_device_status(stream)
        assert out_a.float().abs().max() > 0
        # same kernels, same arithmetic order: identical bits (well inside the 1e-2 / 1e-3 tolerance of the other tests)
        assert torch.equal(out_a, out_b), f"call {call}: max diff {(out_a.float() - out_b.float()).abs().max().item()}"
        assert torch.equal(fin_a, fin_b), f"call {call}"


def test_noalloc_entry_point_rejects_oversized_shapes():
    from quamba_b200 import _lib
    lib = _lib.lib()
    one = torch.zeros(16, dtype=torch.int8, device="cuda")
    a = _lib.make("qb_ssd_args", batch=4, seqlen=2048, nheads=80, headdim=64, ngroups=1, dstate=128, chunk_size=256,
                  x=one.data_ptr())
    rc = lib.qb_ssd_chunk_scan_fwd_noalloc(ctypes.byref(a), None)
    assert rc == _lib.QB_ERR_TOO_LARGE
    assert b"built-in array holds" in lib.qb_last_error()
