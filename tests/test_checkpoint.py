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


# ---- the library's own loader (csrc/checkpoint.cu) against the same fixtures ---------------------
def c_open(lib, path):
    import ctypes as C
    handle = C.c_void_p()
    rc = lib.raw("gemb_checkpoint_open", path.encode(), C.addressof(handle))
    return rc, handle


def test_library_loader_rejects_what_the_reference_rejects(tmp_path, lib):
    """No GPU needed: validation runs before anything touches the device.  Same edits as the Python
    harness's test, and the status codes gem16 reports (kDataLoss for schema violations)."""
    import ctypes as C
    from gem16_b200.lib import STATUS_NAMES

    def nvfp4_bytes(edit):
        mod = fixture_module()
        edit(mod)
        path = str(tmp_path / "c.safetensors")
        write_safetensors(path, mod)
        rc, h = c_open(lib, path)
        assert rc == 0, lib.last_error()
        n = lib.cdll.gemb_checkpoint_nvfp4_bytes(h, b"m")
        rc = lib.raw("gemb_checkpoint_bind_nvfp4", h, b"m", 0, 0, None, 0, None, None) if n == 0 else 0
        lib.gemb_checkpoint_close(h)
        return n, rc

    n, _ = nvfp4_bytes(lambda m: None)
    per = lib.cdll.gemb_interleaved_scale_bytes(8, 64)
    assert n == 256 + 256 + (per + 255) // 256 * 256 + 256 + 256
    for edit, want in ((lambda m: m.pop("m.weight_packed"), "kNotFound"),
                       (lambda m: m.pop("m.weight_scale"), "kDataLoss"),
                       (lambda m: m.pop("m.input_global_scale"), "kDataLoss"),
                       (lambda m: m.__setitem__("m.weight_scale", ("U8", m["m.weight_scale"][1])), "kDataLoss"),
                       (lambda m: m.__setitem__("m.weight_scale", ("F8_E4M3", m["m.weight_scale"][1][:, :3])), "kDataLoss"),
                       (lambda m: m["m.weight_scale"][1].__setitem__((2, 1), 0xFF), "kDataLoss"),
                       (lambda m: m.__setitem__("m.weight_global_scale", ("F32", np.array([0.0], np.float32))), "kDataLoss"),
                       (lambda m: m.__setitem__("m.weight_global_scale", ("BF16", np.array([0x4300], np.uint16))), "kDataLoss"),
                       (lambda m: m.__setitem__("m.input_global_scale", ("F32", np.array(1.0, np.float32))), "kDataLoss"),
                       (lambda m: m.__setitem__("m.weight_packed", ("U8", m["m.weight_packed"][1][:, :24])), "kDataLoss")):
        n, rc = nvfp4_bytes(edit)
        assert n == 0 and STATUS_NAMES[rc] == want, (STATUS_NAMES[rc], lib.last_error())
    # container errors
    bad = str(tmp_path / "bad.safetensors")
    open(bad, "wb").write(b"\x05\x00\x00")
    assert STATUS_NAMES[c_open(lib, bad)[0]] == "kDataLoss"
    assert STATUS_NAMES[c_open(lib, str(tmp_path / "absent.safetensors"))[0]] == "kIoError"
    import json, struct
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    open(bad, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    assert STATUS_NAMES[c_open(lib, bad)[0]] == "kDataLoss"


@pytest.mark.gpu
def test_library_loader_binds_like_the_harness(tmp_path, lib, dev, orc):
    """gemb_checkpoint_bind_nvfp4 / _fp8: the bytes in the arena equal what the Python harness uploads
    (payload, compact and interleaved scales, divisors), for a plain module, an expert stack and an
    FP8 module; the binding then drives the decode GEMV on the pinned checkpoint-byte fixture."""
    import ctypes as C
    from gem16_b200.lib import Fp8Binding, Nvfp4Binding
    rng = np.random.default_rng(5)
    experts, rows, k = 3, 128, 128
    packed = rng.integers(0, 256, (experts, rows, k // 2), dtype=np.uint8)
    scale = rng.integers(0x30, 0x50, (experts, rows, k // 16), dtype=np.uint8)
    wq, wsc = orc.fp8_quantize((rng.standard_normal((40, 528)) * 0.02).astype(np.float32))
    mod = fixture_module()
    mod.update({"x.weight_packed": ("U8", packed), "x.weight_scale": ("F8_E4M3", scale),
                "x.weight_global_scale": ("F32", np.array([100.0, 200.0, 300.0], np.float32)),
                "x.input_global_scale": ("F32", np.array([7.0, 8.0, 9.0], np.float32)),
                "q.weight": ("F8_E4M3", wq), "q.weight_scale": ("BF16", orc.to_bf16(wsc).reshape(-1, 1))})
    path = str(tmp_path / "l.safetensors")
    write_safetensors(path, mod)
    rc, h = c_open(lib, path)
    assert rc == 0
    st = SafetensorsFile(path)
    for name in ("m", "x"):
        want = load_nvfp4_linear(st, name, dev, lib)
        n = lib.cdll.gemb_checkpoint_nvfp4_bytes(h, name.encode())
        arena = torch.zeros((n,), dtype=torch.uint8, device=dev)
        b = Nvfp4Binding()
        lib.gemb_checkpoint_bind_nvfp4(h, name.encode(), want.rows, want.k, arena, n, b, None)
        torch.cuda.synchronize()

        def at(ptr, nbytes):
            off = ptr - arena.data_ptr()
            return arena[off:off + nbytes]

        ne = max(want.experts, 1)
        assert (b.rows, b.contracting, b.experts) == (want.rows, want.k, want.experts)
        assert torch.equal(at(b.packed_weight, want.packed.numel()), want.packed.view(-1))
        assert torch.equal(at(b.scales, want.compact_scales.numel()), want.compact_scales.view(-1))
        assert torch.equal(at(b.scales_interleaved, want.interleaved_scales.numel()), want.interleaved_scales)
        gw = at(b.weight_divisors_device, 4 * ne).view(torch.float32).tolist()
        assert gw == (want.weight_divisor if want.experts else [want.weight_divisor])
        assert b.weight_divisor == gw[0] and at(b.input_divisor_device, 4).view(torch.float32).item() == b.input_divisor
        with pytest.raises(Exception):     # the geometry the model expects must match
            lib.gemb_checkpoint_bind_nvfp4(h, name.encode(), want.rows + 8, want.k, arena, n, b, None)
        if name == "m":                    # pinned bytes of the reference's fixture through the decode GEMV
            act = np.zeros((1, 32), np.uint8)
            act[0, 0] = 2                  # element 0 = 1.0
            y = torch.zeros((8,), device=dev)
            lib.gemb_nvfp4_gemv(torch.from_numpy(act[0]).to(dev), torch.full((4,), 0x38, dtype=torch.uint8, device=dev),
                                b.packed_weight, b.scales, y, 8, 64, 1.0, b.weight_divisor, None)
            assert abs(float(y[0]) - E2M1[FIXTURE_NIBBLES[0]] * FIXTURE_SCALE_VALUE / FIXTURE_DIVISOR) < 1e-9
    n = lib.cdll.gemb_checkpoint_fp8_bytes(h, b"q")
    arena = torch.zeros((n,), dtype=torch.uint8, device=dev)
    f = Fp8Binding()
    lib.gemb_checkpoint_bind_fp8(h, b"q", 40, 528, arena, n, f, None)
    want = load_fp8_linear(st, "q", dev)
    torch.cuda.synchronize()
    assert torch.equal(arena[:40 * 528], want.weight.view(-1)) and (f.rows, f.contracting) == (40, 528)
    off = f.scales - arena.data_ptr()
    assert torch.equal(arena[off:off + 80].view(torch.int16), want.scales_bf16)
    lib.gemb_checkpoint_close(h)
