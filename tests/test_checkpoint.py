"""Checkpoint loader: the safetensors container, the reference's tensor validation rules, and the
reference's pinned checkpoint-byte fixture (tests/unit/nvfp4_test.cpp:104-134) pushed through the real
kernels after loading."""
import numpy as np
import pytest
import torch

from gem16_b200.checkpoint import (CheckpointError, SafetensorsFile, load_fp8_linear, load_nvfp4_linear,
                                   write_safetensors)

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float64)
FIXTURE_PACKED = np.array([0x37, 0xC1, 0x53, 0xA0, 0xFB, 0x5D, 0xAD, 0xFE], np.uint8)
FIXTURE_NIBBLES = [7, 3, 1, 12, 3, 5, 0, 10, 11, 15, 13, 5, 13, 10, 14, 15]
FIXTURE_SCALE, FIXTURE_SCALE_VALUE, FIXTURE_DIVISOR = 0x61, 36.0, 9600.0


def fixture_module(rows=8, k=64, seed=0):
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 256, (rows, k // 2), dtype=np.uint8)
    scale = rng.integers(0x30, 0x50, (rows, k // 16), dtype=np.uint8)
    packed[0, :8] = FIXTURE_PACKED
    scale[0, 0] = FIXTURE_SCALE
    return {"m.weight_packed": ("U8", packed), "m.weight_scale": ("F8_E4M3", scale),
            "m.weight_global_scale": ("F32", np.array([FIXTURE_DIVISOR], np.float32)),
            "m.input_global_scale": ("F32", np.array([1.0], np.float32))}


def test_container_round_trip_and_nibble_order(tmp_path):
    path = str(tmp_path / "a.safetensors")
    mod = fixture_module()
    mod["other.weight_scale"] = ("BF16", np.arange(6, dtype=np.uint16).reshape(6, 1))
    write_safetensors(path, mod, metadata={"format": "pt"})
    st = SafetensorsFile(path)
    assert st.metadata == {"format": "pt"} and set(st.names()) == set(mod)
    for name, (dtype, arr) in mod.items():
        assert st.dtype(name) == dtype and np.array_equal(st.tensor(name), arr)
    # element 2i is the low nibble (src/numeric/nvfp4.cpp:58-70): the fixture's expected nibbles
    p = st.tensor("m.weight_packed")[0, :8]
    assert [int(v) for b in p for v in (b & 15, b >> 4)] == FIXTURE_NIBBLES


def test_container_rejects_malformed_files(tmp_path):
    path = str(tmp_path / "bad.safetensors")
    open(path, "wb").write(b"\x05\x00\x00")
    with pytest.raises(CheckpointError):
        SafetensorsFile(path)
    import json, struct
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    open(path, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(CheckpointError):      # 4 floats cannot be 8 bytes
        SafetensorsFile(path)
    hdr = json.dumps({"t": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 4]}}).encode()
    open(path, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(CheckpointError):
        SafetensorsFile(path)


@pytest.mark.gpu
def test_validation_rules(tmp_path, lib, dev):
    def attempt(edit):
        mod = fixture_module()
        edit(mod)
        path = str(tmp_path / "v.safetensors")
        write_safetensors(path, mod)
        return load_nvfp4_linear(SafetensorsFile(path), "m", dev, lib)

    attempt(lambda m: None)
    for edit in (lambda m: m.pop("m.weight_scale"),
                 lambda m: m.__setitem__("m.weight_scale", ("U8", m["m.weight_scale"][1])),               # wrong dtype
                 lambda m: m.__setitem__("m.weight_scale", ("F8_E4M3", m["m.weight_scale"][1][:, :3])),   # wrong shape
                 lambda m: m["m.weight_scale"][1].__setitem__((2, 1), 0x7F),                              # NaN scale byte
                 lambda m: m.__setitem__("m.weight_global_scale", ("F32", np.array([0.0], np.float32))),  # bad divisor
                 # global scales: both present, F32, shape [1] (src/model/manifest.cpp:346-365).  A BF16 divisor
                 # read as its 16-bit pattern (0x4300 = 128.0 would become 17152.0) would pass a value check.
                 lambda m: m.__setitem__("m.weight_global_scale", ("BF16", np.array([0x4300], np.uint16))),
                 lambda m: m.__setitem__("m.input_global_scale", ("F16", np.array([0x3C00], np.uint16))),
                 lambda m: m.pop("m.input_global_scale"),
                 lambda m: m.pop("m.weight_global_scale"),
                 lambda m: m.__setitem__("m.input_global_scale", ("F32", np.array(1.0, np.float32))),        # shape []
                 lambda m: m.__setitem__("m.weight_global_scale", ("F32", np.array([[9600.0]], np.float32))),  # shape [1, 1]
                 lambda m: m.__setitem__("m.input_global_scale", ("F32", np.array([1.0, 1.0], np.float32))),
                 lambda m: m.__setitem__("m.weight_packed", ("U8", m["m.weight_packed"][1][:, :24]))):    # K = 48
        with pytest.raises(CheckpointError):
            attempt(edit)


@pytest.mark.gpu
def test_pinned_checkpoint_fixture_through_the_kernels(tmp_path, lib, dev):
    """One-hot activations (E2M1 code 2 = 1.0, scale byte 0x38 = 1.0, divisor 1) against the pinned
    bytes of layer 0 Gate row 0: y[0] = decode(nibble) * 36 / 9600, through the decode GEMV on the
    compact scales and through the tcgen05 GEMM on the interleaved ones."""
    path = str(tmp_path / "f.safetensors")
    write_safetensors(path, fixture_module())
    w = load_nvfp4_linear(SafetensorsFile(path), "m", dev, lib)
    assert (w.rows, w.k, w.experts, w.weight_divisor, w.input_divisor) == (8, 64, 0, FIXTURE_DIVISOR, 1.0)
    want = E2M1[FIXTURE_NIBBLES] * FIXTURE_SCALE_VALUE / FIXTURE_DIVISOR
    act = np.zeros((16, 32), np.uint8)
    for sel in range(16):
        act[sel, sel // 2] = 2 << (0 if sel % 2 == 0 else 4)
    act_scales = np.full((16, 4), 0x38, np.uint8)
    a_p, a_s = torch.from_numpy(act).to(dev), torch.from_numpy(act_scales).to(dev)
    got = np.zeros(16)
    for sel in range(16):
        y = torch.zeros((8,), device=dev)
        lib.gemb_nvfp4_gemv(a_p[sel], a_s[sel], w.packed, w.compact_scales, y, 8, 64, 1.0, w.weight_divisor, None)
        got[sel] = float(y[0].item())
    assert np.abs(got - want).max() < 1e-9 + 1e-6 * np.abs(want).max()
    a_inter = torch.zeros((lib.cdll.gemb_interleaved_scale_bytes(16, 64),), dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_interleave_scales(a_s, a_inter, 16, 64, None)
    out = torch.zeros((16, 8), dtype=torch.int16, device=dev)
    lib.gemb_nvfp4_gemm_bf16(a_p, a_inter, w.packed, w.interleaved_scales, out, 16, 8, 64, 1.0, w.weight_divisor, None)
    torch.cuda.synchronize()
    lib.gemb_check_device_status()
    got_mm = out.view(torch.bfloat16).float().cpu().numpy()[:, 0]
    assert np.abs(got_mm - want).max() <= np.abs(want).max() * 2.0 ** -8      # bf16 output rounding


@pytest.mark.gpu
def test_expert_stack_and_fp8_module(tmp_path, lib, dev, orc):
    rng = np.random.default_rng(3)
    experts, rows, k = 3, 128, 128
    packed = rng.integers(0, 256, (experts, rows, k // 2), dtype=np.uint8)
    scale = rng.integers(0x30, 0x50, (experts, rows, k // 16), dtype=np.uint8)
    wf = (rng.standard_normal((40, 528)) * 0.02).astype(np.float32)
    wq, wsc = orc.fp8_quantize(wf)
    path = str(tmp_path / "e.safetensors")
    write_safetensors(path, {"x.weight_packed": ("U8", packed), "x.weight_scale": ("F8_E4M3", scale),
                             "x.weight_global_scale": ("F32", np.array([100.0, 200.0, 300.0], np.float32)),
                             "x.input_global_scale": ("F32", np.array([7.0, 8.0, 9.0], np.float32)),
                             "q.weight": ("F8_E4M3", wq), "q.weight_scale": ("BF16", orc.to_bf16(wsc).reshape(-1, 1))})
    st = SafetensorsFile(path)
    w = load_nvfp4_linear(st, "x", dev, lib)
    assert w.experts == 3 and w.weight_divisor == [100.0, 200.0, 300.0] and w.input_divisor == [7.0, 8.0, 9.0]
    per = lib.cdll.gemb_interleaved_scale_bytes(rows, k)
    got = w.interleaved_scales.cpu().numpy()
    for e in range(experts):
        assert np.array_equal(got[e * per:(e + 1) * per], orc.interleave_scales(scale[e], k))
    f = load_fp8_linear(st, "q", dev)
    x = rng.standard_normal((1, 528)).astype(np.float32)
    xq, xsc = orc.fp8_quantize(x)
    y = torch.zeros((40,), device=dev)
    lib.gemb_fp8_gemv(torch.from_numpy(xq).to(dev), torch.from_numpy(xsc).to(dev), f.weight, f.scales_bf16, y, 40, 528, None)
    want = orc.fp8_matmul(xq, xsc, wq, orc.to_bf16(wsc))[0]
    assert np.linalg.norm(y.cpu().numpy() - want) <= 1e-6 * np.linalg.norm(want)
