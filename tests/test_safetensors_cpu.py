"""CPU suite: the SafeTensors container code of libmft_cuda.so (host only).  Files are produced here byte by byte
with numpy (8-byte header length, JSON header, raw data), in F32 / F16 / BF16, as one file and as a sharded
snapshot with an index, and read back through the C ABI."""
import ctypes as C
import json
import struct

import numpy as np
import pytest


def write_container(path, tensors, metadata=None):
    """tensors: name -> (dtype string, ndarray already in the storage dtype)."""
    header, blobs, off = {}, [], 0
    for name, (dt, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = metadata
    hs = json.dumps(header).encode()
    hs += b" " * (-len(hs) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hs)) + hs + b"".join(blobs))


def bf16_bits(a):
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)


@pytest.fixture(scope="module")
def L():
    from mobilefinetuner_b200 import _lib
    return _lib


def open_(L, path):
    h = C.c_void_p()
    L.call("mft_safetensors_open", str(path).encode(), C.byref(h))
    return h


def read(L, h, name, shape, transpose=False):
    out = np.empty(int(np.prod(shape)), np.float32)
    L.call("mft_safetensors_read_f32", h, name.encode(), out.ctypes.data, 1 if transpose else 0)
    return out


def test_reads_f32_f16_bf16_with_metadata_and_transpose(L, tmp_path):
    g = np.random.Generator(np.random.PCG64(1))
    a = g.standard_normal((5, 7)).astype(np.float32)
    b = g.standard_normal((3, 4)).astype(np.float16)
    c = g.standard_normal((6,)).astype(np.float32)
    c_bits = bf16_bits(c)
    p = tmp_path / "m.safetensors"
    write_container(p, {"w.a": ("F32", a), "w.b": ("F16", b), "w.c": ("BF16", c_bits), "ids": ("I64", np.arange(3))},
                    {"format": "pt", "rank": "8"})
    h = open_(L, p)
    names = sorted(L.call("mft_safetensors_name", h, i).decode() for i in range(L.call("mft_safetensors_count", h)))
    assert names == ["ids", "w.a", "w.b", "w.c"]
    assert L.call("mft_safetensors_metadata", h, b"rank") == b"8" and L.call("mft_safetensors_metadata", h, b"nope") is None
    dt, nd, sh = C.create_string_buffer(8), C.c_int32(), (C.c_int64 * 8)()
    L.call("mft_safetensors_info", h, b"w.b", dt, C.byref(nd), sh)
    assert dt.value == b"F16" and nd.value == 2 and list(sh[:2]) == [3, 4]
    np.testing.assert_array_equal(read(L, h, "w.a", a.shape).reshape(a.shape), a)
    np.testing.assert_array_equal(read(L, h, "w.a", a.shape, transpose=True).reshape(7, 5), a.T)
    np.testing.assert_array_equal(read(L, h, "w.b", b.shape).reshape(b.shape), b.astype(np.float32))
    np.testing.assert_array_equal(read(L, h, "w.c", c.shape), (c_bits.astype(np.uint32) << 16).view(np.float32))
    with pytest.raises(L.MftError):
        read(L, h, "ids", (3,))                      # integer tensors are not weights
    with pytest.raises(L.MftError):
        read(L, h, "missing", (1,))
    L.call("mft_safetensors_close", h)


def test_sharded_snapshot_and_single_file_directory(L, tmp_path):
    g = np.random.Generator(np.random.PCG64(2))
    t = {f"model.layers.{i}.w": g.standard_normal((4, 3)).astype(np.float32) for i in range(4)}
    d = tmp_path / "sharded"
    d.mkdir()
    write_container(d / "model-00001-of-00002.safetensors", {k: ("F32", v) for k, v in list(t.items())[:2]})
    write_container(d / "model-00002-of-00002.safetensors", {k: ("F32", v) for k, v in list(t.items())[2:]})
    index = {"metadata": {"total_size": 192}, "weight_map": {k: ("model-00001-of-00002.safetensors" if i < 2 else "model-00002-of-00002.safetensors")
                                                              for i, k in enumerate(t)}}
    (d / "model.safetensors.index.json").write_text(json.dumps(index))
    h = open_(L, d)
    assert L.call("mft_safetensors_count", h) == 4
    for k, v in t.items():
        np.testing.assert_array_equal(read(L, h, k, v.shape).reshape(v.shape), v)
    L.call("mft_safetensors_close", h)
    d2 = tmp_path / "single"
    d2.mkdir()
    write_container(d2 / "model.safetensors", {"x": ("F32", t["model.layers.0.w"])})
    h = open_(L, d2)
    assert L.call("mft_safetensors_count", h) == 1
    L.call("mft_safetensors_close", h)


def test_writer_output_is_a_valid_sorted_container(L, tmp_path):
    g = np.random.Generator(np.random.PCG64(3))
    arrs = {"layer.1.attn.q.lora_B": g.standard_normal((8, 16)).astype(np.float32),
            "layer.0.attn.q.lora_A": g.standard_normal((16, 8)).astype(np.float32)}
    names = list(arrs)
    n = len(names)
    c_names = (C.c_char_p * n)(*[s.encode() for s in names])
    ndims = (C.c_int32 * n)(2, 2)
    shapes = (C.c_int64 * (8 * n))()
    for i, k in enumerate(names):
        shapes[8 * i], shapes[8 * i + 1] = arrs[k].shape
    data = (C.c_void_p * n)(*[arrs[k].ctypes.data for k in names])
    mk = (C.c_char_p * 2)(b"rank", b"alpha")
    mv = (C.c_char_p * 2)(b"8", b"16")
    p = tmp_path / "adapter.safetensors"
    L.call("mft_safetensors_write_f32", str(p).encode(), n, c_names, ndims, shapes, data, 2, mk, mv)
    raw = p.read_bytes()
    hlen = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + hlen])
    assert hlen % 8 == 0 and header["__metadata__"] == {"rank": "8", "alpha": "16"}
    keys = [k for k in header if k != "__metadata__"]
    assert keys == sorted(names)                                      # sorted, offsets in that order
    assert header[keys[0]]["data_offsets"][0] == 0 and header[keys[1]]["data_offsets"][0] == header[keys[0]]["data_offsets"][1]
    for k in names:
        s0, s1 = header[k]["data_offsets"]
        got = np.frombuffer(raw[8 + hlen + s0: 8 + hlen + s1], np.float32).reshape(header[k]["shape"])
        np.testing.assert_array_equal(got, arrs[k])


def test_rejects_truncated_and_malformed_files(L, tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(L.MftError):
        open_(L, p)
    a = np.zeros((4,), np.float32)
    write_container(p, {"a": ("F32", a)})
    raw = p.read_bytes()
    p.write_bytes(raw[:-8])                                           # data section shorter than data_offsets say
    with pytest.raises(L.MftError):
        open_(L, p)
    with pytest.raises(L.MftError):
        open_(L, tmp_path / "does_not_exist")


def test_cpp_reader_classes_and_key_maps(tmp_path):
    """tests/cpp/safetensors_reader.cpp: SafeTensorsModelReader / SafeTensorsReader / the three key mappers of the
    C++ API, used the way the reference's loading code uses them (host only)."""
    import subprocess
    from mobilefinetuner_b200 import build
    build.build()
    build.build_operators()
    exe = build.build_cpp_tests("safetensors_reader")
    res = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all checks passed" in res.stdout
