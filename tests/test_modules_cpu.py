"""Host logic of the quantized layers that needs no kernel: checkpoint keys, loading, patcher rules."""
import pytest
import torch
import torch.nn as nn


def _fake_nvfp4_state(o=384, i=256, with_input_scale=True):
    g = torch.Generator().manual_seed(0)
    sd = {
        "weight": torch.randint(0, 256, (o, i // 2), generator=g, dtype=torch.uint8),
        "weight_scale": torch.randint(0, 120, (((o + 127) // 128 * 128) * ((i // 16 + 3) // 4 * 4),), generator=g,
                                      dtype=torch.uint8),  # flat bytes, as checkpoints store them
        "weight_scale_2": torch.tensor([0.01]),
        "bias": torch.zeros(o, dtype=torch.bfloat16),
    }
    if with_input_scale:
        sd["input_scale"] = torch.tensor([0.002])
    return sd


def test_nvfp4_linear_loads_and_saves_the_reference_keys():
    from comfy_kitchen.modules import NVFP4Linear
    from comfy_kitchen.tensor import QuantizedTensor

    layer = NVFP4Linear(256, 384)
    sd = _fake_nvfp4_state()
    res = layer.load_state_dict({k: v.clone() for k, v in sd.items()})
    assert not res.missing_keys and not res.unexpected_keys
    assert isinstance(layer.weight, QuantizedTensor) and tuple(layer.weight.shape) == (384, 256)
    assert layer.weight._params.block_scale.dtype == torch.float8_e4m3fn
    assert tuple(layer.weight._params.block_scale.shape) == (384, 16)
    assert layer.input_scale is not None and layer.input_scale.dtype == torch.float32
    out = layer.state_dict()
    assert set(out) == {"weight", "weight_scale", "weight_scale_2", "bias", "input_scale"}
    assert torch.equal(out["weight"], sd["weight"])
    assert torch.equal(out["weight_scale"].view(torch.uint8).reshape(-1), sd["weight_scale"])
    assert float(out["weight_scale_2"]) == pytest.approx(0.01)


def test_nested_prefixes_and_missing_input_scale():
    from comfy_kitchen.modules import NVFP4Linear

    model = nn.ModuleDict({"blk": nn.ModuleDict({"fc": NVFP4Linear(256, 384, bias=False)})})
    sd = {f"blk.fc.{k}": v for k, v in _fake_nvfp4_state(with_input_scale=False).items() if k != "bias"}
    res = model.load_state_dict(sd)
    assert not res.missing_keys and not res.unexpected_keys
    assert model["blk"]["fc"].input_scale is None
    assert set(model.state_dict()) == {"blk.fc.weight", "blk.fc.weight_scale", "blk.fc.weight_scale_2"}


def test_missing_weight_entries_are_reported():
    from comfy_kitchen.modules import MXFP8Linear, NVFP4Linear

    with pytest.raises(RuntimeError, match="weight_scale"):
        NVFP4Linear(256, 384).load_state_dict({"weight": torch.zeros(384, 128, dtype=torch.uint8),
                                               "bias": torch.zeros(384, dtype=torch.bfloat16)})
    with pytest.raises(RuntimeError, match="tiled layout"):
        MXFP8Linear(256, 384).load_state_dict({"weight": torch.zeros(384, 256, dtype=torch.uint8),
                                               "weight_scale": torch.zeros(5, dtype=torch.uint8),
                                               "bias": torch.zeros(384, dtype=torch.bfloat16)})


def test_mxfp8_linear_keys():
    from comfy_kitchen.modules import MXFP8Linear

    layer = MXFP8Linear(256, 384)
    sd = {"weight": torch.zeros(384, 256, dtype=torch.uint8), "weight_scale": torch.full((384 * 8,), 127, dtype=torch.uint8),
          "bias": torch.zeros(384, dtype=torch.bfloat16)}
    res = layer.load_state_dict(sd)
    assert not res.missing_keys and not res.unexpected_keys
    assert layer.weight._qdata.dtype == torch.float8_e4m3fn
    assert layer.weight._params.scale.dtype == torch.float8_e8m0fnu
    assert set(layer.state_dict()) == {"weight", "weight_scale", "bias"}


def test_patcher_rules_on_a_cpu_model():
    from comfy_kitchen.modules import patch_model

    model = nn.Sequential(nn.Linear(128, 256), nn.ReLU(), nn.Linear(256, 16))
    model, report = patch_model(model, layout="mxfp8", skip_names=["0"])
    assert report["patched"] == []
    assert report["skipped"]["0"] == "name matches a skip pattern"
    assert "smaller than" in report["skipped"]["2"]
    model, report = patch_model(nn.Sequential(nn.Linear(128, 256)), layout="nvfp4")
    assert report["skipped"]["0"] == "weight is not on a CUDA device"  # quantization runs on the GPU only
    with pytest.raises(KeyError):
        patch_model(model, layout="int3")


def test_load_follows_the_module_after_it_was_moved():
    """A layer built on the CPU and moved afterwards loads its checkpoint onto the device it is on now
    (the 'meta' device stands in for the GPU here), not the one it was built on."""
    from comfy_kitchen.modules import MXFP8Linear, NVFP4Linear

    layer = NVFP4Linear(256, 384).to("meta")
    assert layer.device.type == "meta"
    res = layer.load_state_dict(_fake_nvfp4_state(), strict=False, assign=False)
    assert not [k for k in res.missing_keys if "bias" not in k]
    assert layer.weight._qdata.device.type == "meta" and layer.weight._params.block_scale.device.type == "meta"
    assert layer.input_scale.device.type == "meta"
    layer8 = MXFP8Linear(256, 384).to("meta")
    layer8.load_state_dict({"weight": torch.zeros(384, 256, dtype=torch.uint8),
                            "weight_scale": torch.full((384 * 8,), 127, dtype=torch.uint8),
                            "bias": torch.zeros(384, dtype=torch.bfloat16)})
    assert layer8.weight._qdata.device.type == "meta"


def test_bias_is_loaded_even_when_the_quantized_entries_are_missing():
    from comfy_kitchen.modules import NVFP4Linear

    layer = NVFP4Linear(256, 384)
    with torch.no_grad():
        layer.bias.zero_()
    res = layer.load_state_dict({"bias": torch.ones(384, dtype=torch.bfloat16)}, strict=False)
    assert set(res.missing_keys) == {"weight", "weight_scale", "weight_scale_2"}
    assert bool((layer.bias == 1).all())


def test_checkpoint_quantizer_selects_the_linear_weights(tmp_path, capsys):
    """The offline quantizer's selection rules and its dry run (no GPU involved)."""
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "comfy-kitchen_b200", "quantize_checkpoint.py")
    spec = importlib.util.spec_from_file_location("quantize_checkpoint", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sd = {"blk.fc1.weight": torch.zeros(256, 128), "blk.fc1.bias": torch.zeros(256), "blk.norm.weight": torch.zeros(128),
          "head.weight": torch.zeros(16, 128), "odd.weight": torch.zeros(128, 72), "emb.weight": torch.zeros(1000, 128, dtype=torch.bfloat16)}
    assert mod.select_keys(sd, 16, 64, [], None) == ["blk.fc1.weight", "emb.weight"]
    assert mod.select_keys(sd, 32, 64, ["emb"], None) == ["blk.fc1.weight"]
    assert mod.select_keys(sd, 16, 64, [], ["head.weight"]) == ["head.weight"]
    with pytest.raises(KeyError):
        mod.select_keys(sd, 16, 64, [], ["nope"])
    ckpt = tmp_path / "m.pt"
    torch.save({"state_dict": sd, "step": 3}, ckpt)
    assert mod.main([str(ckpt), "--dry-run"]) == 0
    assert "2 of 6 entries -> nvfp4" in capsys.readouterr().out
