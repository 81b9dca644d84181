"""Weight ingest: the GGUF reader (host only) and the slab <-> planar conversion (GPU).

The files are written here, once by hand from the published container layout and once with the gguf package's
writer, so the reader is checked against an independent producer."""
import ctypes as C
import struct

import numpy as np
import pytest

from zeromoe_b200 import synth
from zeromoe_b200.lib import GgufTensor

from helpers import to_dev

ERR_ARG, ERR_TYPE, ERR_SHAPE, ERR_STATE = -1, -2, -3, -8
GGUF_TYPE = {synth.Q2_K: 10, synth.Q3_K: 11, synth.Q4_K: 12, synth.IQ2_XXS: 16}


def _gguf_string(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf_by_hand(path, tensors, alignment=32, version=3):
    """tensors: list of (name, ne tuple (ne[0] first), type id, bytes)"""
    kv = [("general.architecture", 8, _gguf_string("zmoe-test")),
          ("general.alignment", 4, struct.pack("<I", alignment)),
          ("test.floats", 9, struct.pack("<IQ", 6, 3) + struct.pack("<3f", 1, 2, 3)),
          ("test.names", 9, struct.pack("<IQ", 8, 2) + _gguf_string("a") + _gguf_string("bc")),
          ("test.flag", 7, b"\x01"), ("test.big", 10, struct.pack("<Q", 1 << 40))]
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv))
    for k, t, payload in kv:
        head += _gguf_string(k) + struct.pack("<I", t) + payload
    off = 0
    blobs = []
    for name, ne, ty, data in tensors:
        head += _gguf_string(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", n) for n in ne)
        head += struct.pack("<IQ", ty, off)
        blobs.append((off, data))
        off += (len(data) + alignment - 1) // alignment * alignment
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        base = f.tell()
        for o, data in blobs:
            f.seek(base + o)
            f.write(data)
        end = f.tell()
        if end < base + off:                      # pad the last tensor to the alignment
            f.write(b"\0" * (base + off - end))


def expert_tensors(seed, layer, E, D, F, types):
    rng = synth.rng_for(seed, layer)
    out = []
    for kind, ty, (O, I) in zip(("gate", "up", "down"), types, ((F, D), (F, D), (D, F))):
        w = synth.random_blocks(ty, E * O * (I // 256), rng).tobytes()
        out.append(("blk.%d.ffn_%s_exps.weight" % (layer, kind), (I, O, E), GGUF_TYPE[ty], w))
    return out


def _open(zlib, path):
    h = C.c_void_p()
    rc = zlib.load().zmoe_gguf_open(str(path).encode(), C.byref(h))
    return rc, h


@pytest.mark.parametrize("alignment", [32, 64])
def test_gguf_reader_hand_written_file(tmp_path, zlib, alignment):
    E, D, F = 4, 512, 256
    types = (synth.Q2_K, synth.Q3_K, synth.Q4_K)
    tensors = [("token_embd.weight", (D, 7), 0, np.arange(7 * D, dtype=np.float32).tobytes())]
    tensors += expert_tensors(11, 0, E, D, F, types) + expert_tensors(11, 3, E, D, F, (synth.IQ2_XXS,) * 3)
    p = tmp_path / "m.gguf"
    write_gguf_by_hand(p, tensors, alignment=alignment)
    rc, h = _open(zlib, p)
    assert rc == 0
    try:
        assert zlib.load().zmoe_gguf_tensor_count(h) == len(tensors)
        for name, ne, ty, data in tensors:
            t = GgufTensor()
            assert zlib.load().zmoe_gguf_find(h, name.encode(), C.byref(t)) == 0
            assert t.type == ty and t.n_dims == len(ne) and tuple(t.ne[:len(ne)]) == ne
            assert t.bytes == len(data) and t.file_offset % alignment == 0
            buf = (C.c_uint8 * len(data))()
            assert zlib.load().zmoe_gguf_read(h, C.byref(t), buf, 0, len(data)) == 0
            assert bytes(buf) == data
            # a window in the middle
            assert zlib.load().zmoe_gguf_read(h, C.byref(t), buf, 100, 50) == 0
            assert bytes(buf[:50]) == data[100:150]
            assert zlib.load().zmoe_gguf_read(h, C.byref(t), buf, len(data) - 10, 11) != 0
        t = GgufTensor()
        assert zlib.load().zmoe_gguf_find(h, b"blk.1.ffn_gate_exps.weight", C.byref(t)) == ERR_STATE
    finally:
        zlib.load().zmoe_gguf_close(h)


def test_gguf_reader_rejects_bad_files(tmp_path, zlib):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGML" + b"\0" * 64)
    rc, h = _open(zlib, p)
    assert rc == ERR_TYPE
    p.write_bytes(b"GGUF" + struct.pack("<IQQ", 1, 0, 0))          # version 1 is not read
    assert _open(zlib, p)[0] == ERR_TYPE
    p.write_bytes(b"GGUF" + struct.pack("<IQQ", 3, 5, 0))          # truncated tensor table
    assert _open(zlib, p)[0] == ERR_SHAPE
    assert _open(zlib, tmp_path / "none.gguf")[0] == ERR_ARG
    # a tensor whose data would lie beyond the end of the file
    good = tmp_path / "short.gguf"
    write_gguf_by_hand(good, expert_tensors(5, 0, 2, 256, 256, (synth.Q4_K,) * 3))
    blob = good.read_bytes()
    good.write_bytes(blob[:len(blob) - 4096])
    rc, h = _open(zlib, good)
    assert rc == 0
    t = GgufTensor()
    assert zlib.load().zmoe_gguf_find(h, b"blk.0.ffn_down_exps.weight", C.byref(t)) == ERR_SHAPE
    zlib.load().zmoe_gguf_close(h)


def test_gguf_reader_file_from_gguf_package(tmp_path, zlib):
    gguf = pytest.importorskip("gguf")
    E, D, F = 3, 256, 512
    p = tmp_path / "w.gguf"
    wr = gguf.GGUFWriter(str(p), "zmoe-test")
    wr.add_uint32("zmoe-test.expert_count", E)
    wr.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])
    datas = {}
    for name, ne, ty, data in expert_tensors(21, 2, E, D, F, (synth.Q2_K, synth.Q4_K, synth.Q3_K)):
        arr = np.frombuffer(data, dtype=np.uint8).reshape(ne[2], ne[1], -1)      # bytes per row innermost
        wr.add_tensor(name, arr, raw_dtype=gguf.GGMLQuantizationType(ty))
        datas[name] = (ne, ty, data)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    rc, h = _open(zlib, p)
    assert rc == 0
    try:
        for name, (ne, ty, data) in datas.items():
            t = GgufTensor()
            assert zlib.load().zmoe_gguf_find(h, name.encode(), C.byref(t)) == 0
            assert t.type == ty and tuple(t.ne[:3]) == ne and t.bytes == len(data)
            buf = (C.c_uint8 * len(data))()
            assert zlib.load().zmoe_gguf_read(h, C.byref(t), buf, 0, len(data)) == 0
            assert bytes(buf) == data
    finally:
        zlib.load().zmoe_gguf_close(h)


def _slab(parts, E):
    per = [len(p) // E for p in parts]
    rec = sum(per)
    stride = (rec + 63) // 64 * 64 + 64
    slab = np.zeros(E * stride, dtype=np.uint8)
    for e in range(E):
        o = e * stride
        for p, n in zip(parts, per):
            slab[o:o + n] = np.frombuffer(p, dtype=np.uint8)[e * n:(e + 1) * n]
            o += n
    return slab, per, stride


@pytest.mark.gpu
@pytest.mark.parametrize("types", [(synth.Q2_K, synth.Q2_K, synth.Q3_K), (synth.IQ2_XXS,) * 3, (synth.Q4_K,) * 3])
def test_unpack_scatter_and_pack_roundtrip(zlib, dev, types):
    import torch
    E, D, F = 6, 512, 768
    parts = [t[3] for t in expert_tensors(31, 0, E, D, F, types)]
    slab, per, stride = _slab(parts, E)
    d_slab = to_dev(slab, dev)
    # planar tensors with a padded per-expert stride
    strides = [n + 32 for n in per]
    planar = [torch.full((E * s,), 0xEE, dtype=torch.uint8, device=dev) for s in strides]
    rc = zlib.load().launch_ggml_moe_unpack(zlib.ptr(d_slab), *[zlib.ptr(p) for p in planar], E, stride, *per, *strides, None)
    assert rc == 0
    torch.cuda.synchronize()
    for p, n, s, src in zip(planar, per, strides, parts):
        got = p.cpu().numpy().reshape(E, s)
        assert np.array_equal(got[:, :n].reshape(-1), np.frombuffer(src, dtype=np.uint8))
        assert (got[:, n:] == 0xEE).all()                     # nothing written past a part
    # scatter: records 0..3 of the slab to slots 5, -1, 0, 2
    slots = np.array([5, -1, 0, 2], dtype=np.int32)
    planar2 = [torch.full((E * s,), 0x11, dtype=torch.uint8, device=dev) for s in strides]
    d_slots = to_dev(slots, dev)
    rc = zlib.load().launch_ggml_moe_unpack_scatter(zlib.ptr(d_slab), *[zlib.ptr(p) for p in planar2], zlib.ptr(d_slots), 4,
                                             stride, *per, *strides, None)
    assert rc == 0
    torch.cuda.synchronize()
    for p, n, s, src in zip(planar2, per, strides, parts):
        got = p.cpu().numpy().reshape(E, s)
        src = np.frombuffer(src, dtype=np.uint8).reshape(E, n)
        for r, slot in enumerate(slots):
            if slot >= 0:
                assert np.array_equal(got[slot, :n], src[r])
        for e in (1, 3, 4):
            assert (got[e] == 0x11).all()
    # and back
    d_back = torch.zeros_like(d_slab)
    rc = zlib.load().zmoe_moe_pack(zlib.ptr(d_back), *[zlib.ptr(p) for p in planar], E, stride, *per, *strides, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(d_back.cpu().numpy(), slab)
    # argument errors come back as a status, nothing is launched
    assert zlib.load().launch_ggml_moe_unpack(None, *[zlib.ptr(p) for p in planar], E, stride, *per, *strides, None) != 0
    assert zlib.load().launch_ggml_moe_unpack_scatter(zlib.ptr(d_slab), *[zlib.ptr(p) for p in planar2], None, 4, stride, *per,
                                               *strides, None) != 0


@pytest.mark.gpu
def test_gguf_load_experts_feeds_the_layer(tmp_path, zlib, oracle, dev):
    """a layer built from tensors loaded out of a GGUF file computes what the oracle computes from the same bytes"""
    import torch
    Context, Layer = zlib.Context, zlib.Layer
    from helpers import routed_inputs, rel_to_norm, REL_TO_NORM
    E, D, F, K, T = 8, 512, 512, 2, 5
    types = (synth.Q2_K, synth.Q2_K, synth.Q3_K)
    tensors = expert_tensors(41, 1, E, D, F, types)
    p = tmp_path / "l.gguf"
    write_gguf_by_hand(p, tensors)
    rc, h = _open(zlib, p)
    assert rc == 0
    bufs = [torch.zeros(len(t[3]), dtype=torch.uint8, device=dev) for t in tensors]
    info = (GgufTensor * 3)()
    assert zlib.load().zmoe_gguf_load_experts(h, 1, *[zlib.ptr(b) for b in bufs], info, None) == 0
    assert zlib.load().zmoe_gguf_load_experts(h, 0, *[zlib.ptr(b) for b in bufs], info, None) == ERR_STATE
    zlib.load().zmoe_gguf_close(h)
    for b, t in zip(bufs, tensors):
        assert bytes(b.cpu().numpy()) == t[3]
    assert [i.type for i in info] == [GGUF_TYPE[t] for t in types]
    wr, x, probs, ids, w = routed_inputs(oracle, 77, T, D, E, K)
    ws = [np.frombuffer(t[3], dtype=np.uint8) for t in tensors]
    ref = oracle.moe_ffn(oracle.make_layer(D, F, E, K, types, ws[0], ws[1], ws[2]), x, ids, w)
    ctx = Context(16, D, F, E, K)
    layer = Layer(ctx, D, F, E, K, types, *[b.view(E, -1) for b in bufs], router_w=to_dev(wr, dev))
    out = torch.zeros(T, D, dtype=torch.float32, device=dev)
    layer.forward(to_dev(x, dev), out)
    torch.cuda.synchronize()
    assert rel_to_norm(out.cpu().numpy(), ref) < REL_TO_NORM
    layer.close(); ctx.close()
