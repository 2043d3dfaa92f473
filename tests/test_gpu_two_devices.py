"""One process driving two GPUs: kernel attributes (dynamic shared memory above 48 KB), constant tables, the device status
word and the static scratch belong to a device, so the first launch on the second device must set them up again.  Every op
runs on cuda:0, then on cuda:1, and the results must be identical.  Skipped with fewer than two GPUs."""
import pytest
import torch

from helpers import make_conv2_case, make_ssd_case

pytestmark = pytest.mark.gpu


def _two():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def _run_everything(dev):
    from quamba_b200 import _lib, ops
    from quamba_b200.modules import W4A8B16O16Linear
    torch.cuda.set_device(dev)
    to = lambda t: None if t is None else t.to(dev)
    out = {}
    g = torch.Generator().manual_seed(0)
    # tensor-core Hadamard (64 KB+ of dynamic shared memory) and the SIMT one
    x = torch.randn(300, 5120, generator=g).half()
    out["had40"] = ops.quant_hadamard.fast_hadamard_transform_40N(to(x), 0.3)
    out["had_pow2"] = ops.quant_hadamard.fast_hadamard_transform(to(x[:, :4096].contiguous()), 0.3)
    # persistent GEMM + decode-sized products on one packed weight
    lin = torch.nn.Linear(2560, 5120, bias=False)
    lin.weight.data = torch.randn(5120, 2560, generator=g) * 0.02
    lin.w4_group_size = -1
    ql = W4A8B16O16Linear.from_fp16(lin, torch.tensor(0.02)).to(dev)
    a = torch.randint(-127, 128, (4096, 2560), generator=g, dtype=torch.int32).to(torch.int8)
    out["gemm"] = ql(to(a))
    out["gemv"] = ql(to(a[:1]))
    out["decode_linear"] = ops.decode_linear(to(a[:2]).contiguous(), ql.prepared(), ql.input_scale)
    # SSD chunk scan (tcgen05 path) and the Mamba2 state update (warp kernel: 64 KB ring)
    s = make_ssd_case(2, 300, 8, 64, 1, 128, 256, seed=1)
    y, f = ops._quant_mamba_chunk_scan_combined_fwd(to(s["q_x"]), to(s["x_scales"]), to(s["q_dt"]), to(s["s_dt"]), to(s["q_A_log"]),
                                                    to(s["s_A"]), to(s["q_B"]), to(s["s_B"]), to(s["q_C"]), to(s["s_C"]), to(s["state_scale"]),
                                                    256, to(s["q_D"]), to(s["s_D"]), None, None, to(s["dt_bias"]), None, None, None, True)
    out["ssd_y"], out["ssd_state"] = y, f
    state = f.clone()
    yy = ops.quant_sscan_update_triton(state, to(s["q_x"][:, 0].contiguous()), to(s["x_scales"]),
                                       to(s["q_dt"][:, 0, :, None].expand(-1, -1, 64)), to(s["s_dt"]),
                                       to(s["q_A_log"][:, None, None].expand(-1, 64, 128)), to(s["s_A"]), to(s["state_scale"]),
                                       to(s["q_B"][:, 0]), to(s["s_B"]), to(s["q_C"][:, 0]), to(s["s_C"]), None, None, None, None,
                                       to(s["dt_bias"][:, None].expand(-1, 64)), None, True)
    out["update_y"], out["update_state"] = yy, state
    # conv
    c = make_conv2_case(1, 130, 8, 64, 1, 128, seed=2)
    xBC = c["xBC"].transpose(1, 2).contiguous().to(dev).transpose(1, 2)
    got = ops.quamba2_conv1d_cuda.fwd(xBC, c["sx"], c["sB"], c["sC"], c["x_dim"], 64, 128, 1, None, None, to(c["x_scales"]), to(c["B_scales"]),
                                      to(c["C_scales"]), to(c["weight"]), c["swx"], c["swB"], c["swC"], to(c["bias"]), c["sbx"], c["sbB"],
                                      c["sbC"], None, None, None, True)
    out["conv_x"], out["conv_B"], out["conv_C"] = got
    torch.cuda.synchronize(dev)
    _lib.read_device_status(torch.cuda.current_stream(dev).cuda_stream)
    return {k: v.cpu() for k, v in out.items()}


def test_every_op_on_the_second_device_after_the_first():
    _two()
    first = _run_everything(torch.device("cuda", 0))
    second = _run_everything(torch.device("cuda", 1))
    again = _run_everything(torch.device("cuda", 0))
    for k in first:
        assert torch.equal(first[k], second[k]), f"{k}: cuda:1 differs from cuda:0"
        assert torch.equal(first[k], again[k]), f"{k}: cuda:0 differs after cuda:1 was used"
    torch.cuda.set_device(0)
