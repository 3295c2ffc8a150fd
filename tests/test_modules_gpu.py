"""Quantized nn.Linear replacements, model patcher and offline weight quantizer
(reference behaviour: samples/nvfp4_linear.py, samples/mxfp8_model_patcher.py)."""
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ck(cuda_device):
    import comfy_kitchen

    info = comfy_kitchen.list_backends()["cuda"]
    assert info["available"], f"cuda backend not loaded: {info['unavailable_reason']}"
    return comfy_kitchen


def _dense(cuda_device, i=256, o=384, bias=True, seed=0):
    torch.manual_seed(seed)
    lin = nn.Linear(i, o, bias=bias, device=cuda_device, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.mul_(0.5)
    return lin


def test_nvfp4_linear_equals_the_operator_sequence(ck, cuda_device):
    from comfy_kitchen.modules import NVFP4Linear

    lin = _dense(cuda_device)
    q = NVFP4Linear.from_linear(lin)
    x = torch.randn(96, 256, device=cuda_device, dtype=torch.bfloat16)
    with torch.inference_mode():
        y = q(x)
    sx = (x.abs().amax() / 2688).float()
    sw = (lin.weight.detach().abs().amax() / 2688).float()
    qx, bsx = ck.quantize_nvfp4(x, sx)
    qw, bsw = ck.quantize_nvfp4(lin.weight.detach(), sw)
    ref = ck.scaled_mm_nvfp4(qx, qw, sx, sw, bsx, bsw, bias=lin.bias.detach(), out_dtype=torch.bfloat16)
    assert torch.equal(y, ref)
    dense = lin(x)
    rel = ((y.float() - dense.float()).norm() / dense.float().norm()).item()
    assert rel < 0.2  # FP4 quantization error of both operands, not a kernel tolerance


def test_nvfp4_linear_state_dict_round_trip_and_keys(ck, cuda_device):
    from comfy_kitchen.modules import NVFP4Linear

    lin = _dense(cuda_device)
    q = NVFP4Linear.from_linear(lin, input_scale=0.004)
    sd = q.state_dict()
    assert set(sd) == {"weight", "weight_scale", "weight_scale_2", "bias", "input_scale"}
    assert sd["weight"].dtype == torch.uint8 and tuple(sd["weight"].shape) == (384, 128)
    # block scales may be stored as raw bytes (float8 support in checkpoint formats is spotty)
    sd["weight_scale"] = sd["weight_scale"].view(torch.uint8).reshape(-1).cpu()
    fresh = NVFP4Linear(256, 384, device=cuda_device, dtype=torch.bfloat16)
    result = fresh.load_state_dict({k: v.clone() for k, v in sd.items()})
    assert not result.missing_keys and not result.unexpected_keys
    x = torch.randn(4, 40, 256, device=cuda_device, dtype=torch.bfloat16)  # 3-D input
    with torch.inference_mode():
        a, b = q(x), fresh(x)
    assert a.shape == (4, 40, 384)
    assert torch.equal(a, b)


def test_nvfp4_linear_without_input_scale_is_dynamic(ck, cuda_device):
    from comfy_kitchen.modules import NVFP4Linear

    q = NVFP4Linear.from_linear(_dense(cuda_device, bias=False))
    sd = q.state_dict()
    assert "input_scale" not in sd and "bias" not in sd
    fresh = NVFP4Linear(256, 384, bias=False, device=cuda_device, dtype=torch.bfloat16)
    fresh.load_state_dict(sd)
    assert fresh.input_scale is None
    x = torch.randn(32, 256, device=cuda_device, dtype=torch.bfloat16)
    with torch.inference_mode():
        assert torch.equal(q(x), fresh(x))


def test_load_reports_missing_and_malformed_entries(ck, cuda_device):
    from comfy_kitchen.modules import NVFP4Linear

    fresh = NVFP4Linear(256, 384, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="weight_scale_2"):
        fresh.load_state_dict({"weight": torch.zeros(384, 128, dtype=torch.uint8),
                               "weight_scale": torch.zeros(384 * 16, dtype=torch.uint8),
                               "bias": torch.zeros(384, dtype=torch.bfloat16)})
    with pytest.raises(RuntimeError, match="tiled layout"):
        fresh.load_state_dict({"weight": torch.zeros(384, 128, dtype=torch.uint8),
                               "weight_scale": torch.zeros(7, dtype=torch.uint8),
                               "weight_scale_2": torch.ones(1), "bias": torch.zeros(384, dtype=torch.bfloat16)})


def test_mxfp8_linear_round_trip(ck, cuda_device):
    from comfy_kitchen.modules import MXFP8Linear

    lin = _dense(cuda_device)
    q = MXFP8Linear.from_linear(lin)
    sd = q.state_dict()
    assert set(sd) == {"weight", "weight_scale", "bias"}
    fresh = MXFP8Linear(256, 384, device=cuda_device, dtype=torch.bfloat16)
    fresh.load_state_dict({k: (v.view(torch.uint8) if k != "bias" else v) for k, v in sd.items()})
    x = torch.randn(2, 33, 256, device=cuda_device, dtype=torch.bfloat16)
    with torch.inference_mode():
        a, b = q(x), fresh(x)
    assert torch.equal(a, b) and a.shape == (2, 33, 384)
    qx, bsx = ck.quantize_mxfp8(x.reshape(-1, 256), pad_32x=True)
    qw, bsw = ck.quantize_mxfp8(lin.weight.detach())
    ref = ck.scaled_mm_mxfp8(qx, qw, bsx, bsw, bias=lin.bias.detach(), out_dtype=torch.bfloat16)[:66]
    assert torch.equal(a.reshape(-1, 384), ref)


class _Tiny(nn.Module):
    def __init__(self, dev):
        super().__init__()
        kw = dict(device=dev, dtype=torch.bfloat16)
        self.inp = nn.Linear(128, 256, **kw)
        self.blocks = nn.ModuleList([nn.Sequential(nn.Linear(256, 512, **kw), nn.GELU(approximate="tanh"),
                                                   nn.Linear(512, 256, **kw)) for _ in range(2)])
        self.head = nn.Linear(256, 24, **kw)   # too small
        self.odd = nn.Linear(200, 256, **kw)   # in_features % 32 != 0 (but % 16 != 0 too: 200 % 16 = 8)

    def forward(self, x):
        x = self.inp(x)
        for b in self.blocks:
            x = x + b(x)
        return self.head(x)


@pytest.mark.parametrize("layout", ["nvfp4", "mxfp8"])
def test_patch_model(ck, cuda_device, layout):
    from comfy_kitchen.modules import MXFP8Linear, NVFP4Linear, patch_model

    torch.manual_seed(1)
    model = _Tiny(cuda_device)
    x = torch.randn(3, 50, 128, device=cuda_device, dtype=torch.bfloat16)
    dense = model(x)
    model, report = patch_model(model, layout=layout, skip_names=["blocks.1.2"])
    cls = NVFP4Linear if layout == "nvfp4" else MXFP8Linear
    assert isinstance(model.inp, cls) and isinstance(model.blocks[0][0], cls) and isinstance(model.blocks[1][0], cls)
    assert isinstance(model.blocks[1][2], nn.Linear) and isinstance(model.head, nn.Linear) and isinstance(model.odd, nn.Linear)
    assert sorted(report["patched"]) == ["blocks.0.0", "blocks.0.2", "blocks.1.0", "inp"]
    assert set(report["skipped"]) == {"blocks.1.2", "head", "odd"}
    with torch.inference_mode():
        y = model(x)
    assert y.shape == dense.shape
    rel = ((y.float() - dense.float()).norm() / dense.float().norm()).item()
    assert rel < (0.35 if layout == "nvfp4" else 0.1)


def test_quantize_state_dict_feeds_the_layer(ck, cuda_device):
    from comfy_kitchen.modules import NVFP4Linear, quantize_state_dict

    lin = _dense(cuda_device)
    sd = quantize_state_dict({"fc.weight": lin.weight.detach().cpu(), "fc.bias": lin.bias.detach().cpu(),
                              "norm.weight": torch.ones(256)}, layout="nvfp4", device=cuda_device)
    assert set(sd) == {"fc.weight", "fc.weight_scale", "fc.weight_scale_2", "fc.bias", "norm.weight"}
    assert sd["fc.weight_scale"].dtype == torch.uint8 and not sd["fc.weight"].is_cuda
    holder = nn.ModuleDict({"fc": NVFP4Linear(256, 384, device=cuda_device, dtype=torch.bfloat16)})
    holder.load_state_dict({k: v for k, v in sd.items() if k.startswith("fc.")})
    x = torch.randn(64, 256, device=cuda_device, dtype=torch.bfloat16)
    with torch.inference_mode():
        assert torch.equal(holder["fc"](x), NVFP4Linear.from_linear(lin)(x))


def test_mmdit_shaped_stack_runs_quantized(ck, cuda_device):
    """The full-model harness of the benchmark at toy size: every block linear through NVFP4, output
    finite and close to the same stack with dense linears."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench_mmdit as mm
    from comfy_kitchen.modules import NVFP4Linear

    cfg = mm.MMDiTConfig(hidden=256, heads=2, double_blocks=1, single_blocks=2, mlp_ratio=4, img_tokens=96, txt_tokens=32)
    assert cfg.linear_params == (1 * 36 + 2 * 15) * 256 * 256
    with torch.inference_mode():
        dense = mm.MMDiTStack(cfg, cuda_device, lambda lin: lin, seed=3)
        quant = mm.MMDiTStack(cfg, cuda_device, NVFP4Linear.from_linear, seed=3)
        img, txt, vec = mm.make_inputs(cfg, 2, cuda_device)
        a, b = dense(img, txt, vec), quant(img, txt, vec)
    assert b.shape == (2, 96, 256) and torch.isfinite(b.float()).all()
    assert all(isinstance(m, NVFP4Linear) for m in quant.modules() if hasattr(m, "in_features"))
    rel = ((a.float() - b.float()).norm() / a.float().norm()).item()
    assert rel < 0.3


def test_checkpoint_quantizer_cli_round_trip(ck, cuda_device, tmp_path):
    """quantize_checkpoint.py on a saved dense model: the output loads into the quantized layers and
    gives the result of quantizing the live layer."""
    import importlib.util
    import os

    from comfy_kitchen.modules import NVFP4Linear

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "comfy-kitchen_b200", "quantize_checkpoint.py")
    spec = importlib.util.spec_from_file_location("quantize_checkpoint", path)
    cli = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cli)
    lin = _dense(cuda_device)
    src, dst = tmp_path / "dense.pt", tmp_path / "q.pt"
    torch.save({k: v.cpu() for k, v in lin.state_dict().items()}, src)
    assert cli.main([str(src), str(dst), "--layout", "nvfp4", "--device", str(cuda_device)]) == 0
    sd = torch.load(dst, map_location="cpu", weights_only=True)
    assert set(sd) == {"weight", "weight_scale", "weight_scale_2", "bias"} and sd["weight"].dtype == torch.uint8
    layer = NVFP4Linear(256, 384, device=cuda_device)
    layer.load_state_dict(sd)
    x = torch.randn(64, 256, device=cuda_device, dtype=torch.bfloat16)
    with torch.inference_mode():
        assert torch.equal(layer(x), NVFP4Linear.from_linear(lin)(x))


def test_captured_graph_survives_growth_of_the_cached_scratch_buffers(ck, cuda_device):
    """The wrappers cache scratch / workspace buffers per stream and replace them when a larger input
    comes along; a CUDA graph captured before still points at the old buffer, which therefore has to
    stay alive (and zeroed where the kernels expect zeros)."""
    from comfy_kitchen.backends import cuda as backend
    from comfy_kitchen.tensor import QuantizedTensor

    side = torch.cuda.Stream()
    x = torch.randn(64, 256, device=cuda_device, dtype=torch.bfloat16)
    w = QuantizedTensor.from_float(torch.randn(128, 256, device=cuda_device, dtype=torch.bfloat16), "TensorCoreNVFP4Layout")
    with torch.cuda.stream(side), torch.inference_mode():
        key = (cuda_device, side.cuda_stream)

        def step():
            return torch.nn.functional.linear(QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout"), w)

        eager = step()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y = step()
        old = backend._scale_scratch[key]
        # a request beyond the cached size replaces the buffer; the captured graph keeps using the old one
        backend._scale_scratch_for(cuda_device, side.cuda_stream, old.numel() * 2)
        assert backend._scale_scratch[key] is not old and any(t is old for t in backend._retired_workspaces)
        torch.nn.functional.linear(QuantizedTensor.from_float(x * 2, "TensorCoreNVFP4Layout"), w)  # uses the new buffer
        for _ in range(2):
            graph.replay()
            side.synchronize()
            assert torch.equal(y, eager)


@pytest.mark.parametrize("rows", [200, 77])  # 77: rows padded to 16 inside the quantizer
def test_nvfp4_mlp_fused_equals_the_unfused_layers(ck, cuda_device, rows):
    """fc1 -> GELU -> quantize (static scale) -> fc2 with the middle steps in fc1's epilogue: same bits."""
    from comfy_kitchen.modules import NVFP4Linear, NVFP4MLP

    fc1 = NVFP4Linear.from_linear(_dense(cuda_device, 256, 512, seed=1))
    fc2 = NVFP4Linear.from_linear(_dense(cuda_device, 512, 256, seed=2))
    mlp = NVFP4MLP(fc1, fc2)
    x = torch.randn(2, rows // 2 if rows % 2 == 0 else rows, 256, device=cuda_device, dtype=torch.bfloat16)
    x = x[:1] if rows % 2 else x  # [1, 77, 256] or [2, 100, 256]
    with torch.inference_mode():
        assert not mlp.fusable()
        dynamic = mlp(x)  # no static scale yet: plain layers, dynamic hidden scale
        assert torch.equal(dynamic, fc2(torch.nn.functional.gelu(fc1(x), approximate="tanh")))
        scale = mlp.calibrate(x)
        assert mlp.fusable() and float(scale) > 0
        fused = mlp(x)
        unfused = fc2(torch.nn.functional.gelu(fc1(x), approximate="tanh"))  # fc2 now quantizes against the static scale
    assert fused.shape == unfused.shape == (*x.shape[:-1], 256)
    assert torch.equal(fused, unfused)
    assert "fc2.input_scale" in mlp.state_dict()


def test_layers_replay_from_a_cuda_graph(ck, cuda_device):
    """The one-call paths of the layers and the fused MLP are launch-only: captured once, replayed on
    new input values, same bits as the eager call."""
    from comfy_kitchen.modules import MXFP8Linear, NVFP4Linear, NVFP4MLP

    fc1 = NVFP4Linear.from_linear(_dense(cuda_device, 256, 512, seed=3))
    fc2 = NVFP4Linear.from_linear(_dense(cuda_device, 512, 256, seed=4))
    mlp = NVFP4MLP(fc1, fc2)
    mx = MXFP8Linear.from_linear(_dense(cuda_device, 256, 384, seed=5))
    x = torch.randn(160, 256, device=cuda_device, dtype=torch.bfloat16)
    with torch.inference_mode():
        mlp.calibrate(x)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up on the capture stream: workspaces are per stream
                mlp(x), fc1(x), mx(x)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                outs = (mlp(x), fc1(x), mx(x))
        x.copy_(torch.randn(160, 256, device=cuda_device, dtype=torch.bfloat16))
        graph.replay()
        torch.cuda.synchronize()
        want = (mlp(x), fc1(x), mx(x))
    for got, ref in zip(outs, want):
        assert torch.equal(got, ref)
