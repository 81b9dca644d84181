// ingest.cu -- weight ingest for the expert path: a reader of the GGUF container that locates a layer's
// expert tensors, and the device-side conversion between the expert-major [gate|up|down] slab and the three
// planar tensors.
//
// Replaces reference kernels/math/ggml_moe_pack.cu:13-179 (launch_ggml_moe_unpack, launch_ggml_moe_unpack_scatter:
// same signatures and meaning) and the part of reference models/base/gguf_loader.hpp that finds
// blk.N.ffn_{gate,up,down}_exps.weight, their GGUFType (:28-51) and their offsets.  The container layout read
// here is the published GGUF format (versions 2 and 3): magic, version, tensor count, key/value count,
// key/values, tensor infos (name, dims, type, offset), padding to general.alignment (default 32), data.
// Note that the library's layer entry takes slabs as they are (a per-expert stride per tensor), so the
// unpack is only needed by hosts that keep planar ggml tensors.
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "zmoe_common.cuh"
#include "zmoe_internal.h"

using namespace zmoe;

namespace {

// One CTA per (record, part, chunk of the part): 16-byte copies where source and destination allow, bytes for
// the ragged ends.  slots == nullptr: record i goes to expert i; otherwise to expert slots[i] (negative: skipped).
// TO_SLAB: the opposite direction.
template <bool TO_SLAB>
__global__ void __launch_bounds__(256) moe_repack_kernel(uint8_t *__restrict__ slab, uint8_t *__restrict__ gate,
                                                         uint8_t *__restrict__ up, uint8_t *__restrict__ down,
                                                         const int32_t *__restrict__ slots, size_t slab_stride,
                                                         size_t gate_bytes, size_t up_bytes, size_t down_bytes,
                                                         size_t gate_stride, size_t up_stride, size_t down_stride,
                                                         int chunks) {
    const int rec = blockIdx.x, part = blockIdx.y, chunk = blockIdx.z;
    const int expert = slots ? slots[rec] : rec;
    if (expert < 0) return;
    const size_t bytes = part == 0 ? gate_bytes : part == 1 ? up_bytes : down_bytes;
    const size_t off_in_slab = part == 0 ? 0 : part == 1 ? gate_bytes : gate_bytes + up_bytes;
    uint8_t *planar = (part == 0 ? gate + (size_t)expert * gate_stride
                                 : part == 1 ? up + (size_t)expert * up_stride : down + (size_t)expert * down_stride);
    uint8_t *in_slab = slab + (size_t)rec * slab_stride + off_in_slab;
    uint8_t *dst = TO_SLAB ? in_slab : planar;
    const uint8_t *src = TO_SLAB ? planar : in_slab;
    const size_t per = ((bytes + chunks - 1) / chunks + 15) & ~(size_t)15;
    const size_t b0 = (size_t)chunk * per, b1 = b0 + per < bytes ? b0 + per : bytes;
    if (b0 >= b1) return;
    if ((((uintptr_t)(dst + b0) | (uintptr_t)(src + b0)) & 15) == 0) {
        const size_t n16 = (b1 - b0) / 16;
        for (size_t i = threadIdx.x; i < n16; i += blockDim.x)
            reinterpret_cast<uint4 *>(dst + b0)[i] = reinterpret_cast<const uint4 *>(src + b0)[i];
        for (size_t i = b0 + 16 * n16 + threadIdx.x; i < b1; i += blockDim.x) dst[i] = src[i];
    } else {
        for (size_t i = b0 + threadIdx.x; i < b1; i += blockDim.x) dst[i] = src[i];
    }
}

template <bool TO_SLAB>
int repack(void *slab, void *gate, void *up, void *down, const int32_t *slots, int count, size_t slab_stride,
           size_t gate_bytes, size_t up_bytes, size_t down_bytes, size_t gate_stride, size_t up_stride,
           size_t down_stride, cudaStream_t st) {
    if (!slab || !gate || !up || !down || count <= 0) return (int)cudaErrorInvalidValue;
    size_t big = gate_bytes > up_bytes ? gate_bytes : up_bytes;
    if (down_bytes > big) big = down_bytes;
    int chunks = 1;
    const int n_sm = device_sm_count();
    while ((long)count * 3 * chunks < 2L * n_sm && big / (chunks * 2) >= 16384) chunks *= 2;
    moe_repack_kernel<TO_SLAB><<<dim3(count, 3, chunks), 256, 0, st>>>(
        static_cast<uint8_t *>(slab), static_cast<uint8_t *>(gate), static_cast<uint8_t *>(up), static_cast<uint8_t *>(down),
        slots, slab_stride, gate_bytes, up_bytes, down_bytes, gate_stride, up_stride, down_stride, chunks);
    count_launches(1);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// GGUF reader (host)
// ---------------------------------------------------------------------------
struct TensorInfo {
    std::string name;
    uint32_t type = 0;
    uint64_t ne[4] = {1, 1, 1, 1};
    int n_dims = 0;
    uint64_t offset = 0;   // from the start of the data section
};

struct Reader {
    FILE *f = nullptr;
    bool ok = true;
    template <typename T> T get() {
        T v{};
        if (ok && fread(&v, sizeof(T), 1, f) != 1) ok = false;
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (1u << 20)) { ok = false; return std::string(); }
        std::string s(n, '\0');
        if (n && fread(&s[0], 1, n, f) != n) ok = false;
        return s;
    }
    void skip(uint64_t n) { if (ok && fseek(f, (long)n, SEEK_CUR) != 0) ok = false; }
};

// sizes of the scalar value types of the key/value section (GGUF value type ids 0..12; 8 = string, 9 = array)
size_t scalar_size(uint32_t t) {
    switch (t) {
    case 0: case 1: case 7: return 1;   // u8, i8, bool
    case 2: case 3: return 2;           // u16, i16
    case 4: case 5: case 6: return 4;   // u32, i32, f32
    case 10: case 11: case 12: return 8; // u64, i64, f64
    }
    return 0;
}

bool skip_value(Reader &r, uint32_t t) {
    if (t == 8) { r.str(); return r.ok; }
    if (t == 9) {
        const uint32_t et = r.get<uint32_t>();
        const uint64_t n = r.get<uint64_t>();
        if (!r.ok) return false;
        if (et == 8) { for (uint64_t i = 0; i < n && r.ok; ++i) r.str(); return r.ok; }
        const size_t sz = scalar_size(et);
        if (!sz) return false;
        r.skip(n * sz);
        return r.ok;
    }
    const size_t sz = scalar_size(t);
    if (!sz) return false;
    r.skip(sz);
    return r.ok;
}

}  // namespace

struct zmoe_gguf {
    FILE *f = nullptr;
    uint64_t data_start = 0, file_bytes = 0;
    std::vector<TensorInfo> tensors;
};

extern "C" {

int launch_ggml_moe_unpack(const void *src, void *gate, void *up, void *down, int count, size_t src_stride,
                           size_t gate_bytes, size_t up_bytes, size_t down_bytes, size_t gate_stride, size_t up_stride,
                           size_t down_stride, void *stream) {
    return repack<false>(const_cast<void *>(src), gate, up, down, nullptr, count, src_stride, gate_bytes, up_bytes, down_bytes,
                         gate_stride, up_stride, down_stride, static_cast<cudaStream_t>(stream));
}

int launch_ggml_moe_unpack_scatter(const void *src, void *gate, void *up, void *down, const int32_t *dst_slots, int count,
                                   size_t src_stride, size_t gate_bytes, size_t up_bytes, size_t down_bytes,
                                   size_t gate_stride, size_t up_stride, size_t down_stride, void *stream) {
    if (!dst_slots) return (int)cudaErrorInvalidValue;
    return repack<false>(const_cast<void *>(src), gate, up, down, dst_slots, count, src_stride, gate_bytes, up_bytes,
                         down_bytes, gate_stride, up_stride, down_stride, static_cast<cudaStream_t>(stream));
}

int zmoe_moe_pack(void *slab, const void *gate, const void *up, const void *down, int count, size_t slab_stride,
                  size_t gate_bytes, size_t up_bytes, size_t down_bytes, size_t gate_stride, size_t up_stride,
                  size_t down_stride, void *stream) {
    return repack<true>(slab, const_cast<void *>(gate), const_cast<void *>(up), const_cast<void *>(down), nullptr, count,
                        slab_stride, gate_bytes, up_bytes, down_bytes, gate_stride, up_stride, down_stride,
                        static_cast<cudaStream_t>(stream));
}

void zmoe_gguf_close(zmoe_gguf *g) {
    if (!g) return;
    if (g->f) fclose(g->f);
    delete g;
}

int zmoe_gguf_open(const char *path, zmoe_gguf **out) {
    if (!path || !out) return ZMOE_ERR_ARG;
    zmoe_gguf *g = new (std::nothrow) zmoe_gguf();
    if (!g) return ZMOE_ERR_ARG;
    g->f = fopen(path, "rb");
    if (!g->f) { delete g; return ZMOE_ERR_ARG; }
    Reader r;
    r.f = g->f;
    char magic[4] = {0, 0, 0, 0};
    if (fread(magic, 1, 4, g->f) != 4 || memcmp(magic, "GGUF", 4) != 0) { zmoe_gguf_close(g); return ZMOE_ERR_TYPE; }
    const uint32_t version = r.get<uint32_t>();
    if (version != 2 && version != 3) { zmoe_gguf_close(g); return ZMOE_ERR_TYPE; }
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    uint64_t alignment = 32;
    for (uint64_t i = 0; i < n_kv && r.ok; ++i) {
        const std::string key = r.str();
        const uint32_t t = r.get<uint32_t>();
        if (key == "general.alignment" && t == 4) alignment = r.get<uint32_t>();
        else if (!skip_value(r, t)) r.ok = false;
    }
    for (uint64_t i = 0; i < n_tensors && r.ok; ++i) {
        TensorInfo ti;
        ti.name = r.str();
        ti.n_dims = (int)r.get<uint32_t>();
        if (ti.n_dims < 1 || ti.n_dims > 4) { r.ok = false; break; }
        for (int d = 0; d < ti.n_dims; ++d) ti.ne[d] = r.get<uint64_t>();
        ti.type = r.get<uint32_t>();
        ti.offset = r.get<uint64_t>();
        g->tensors.push_back(ti);
    }
    if (!r.ok || alignment == 0) { zmoe_gguf_close(g); return ZMOE_ERR_SHAPE; }
    const long here = ftell(g->f);
    g->data_start = ((uint64_t)here + alignment - 1) / alignment * alignment;
    fseek(g->f, 0, SEEK_END);
    g->file_bytes = (uint64_t)ftell(g->f);
    *out = g;
    return ZMOE_OK;
}

int zmoe_gguf_tensor_count(zmoe_gguf *g) { return g ? (int)g->tensors.size() : 0; }

int zmoe_gguf_find(zmoe_gguf *g, const char *name, zmoe_gguf_tensor *out) {
    if (!g || !name || !out) return ZMOE_ERR_ARG;
    for (const TensorInfo &t : g->tensors) {
        if (t.name != name) continue;
        out->type = (int)t.type;
        out->n_dims = t.n_dims;
        for (int d = 0; d < 4; ++d) out->ne[d] = (int64_t)t.ne[d];
        out->file_offset = g->data_start + t.offset;
        // bytes: rows of ne[0] elements in blocks of the type
        const int bb = t.type == 8 ? 34 : block_bytes((int)t.type);
        const uint64_t per = t.type == 8 ? 32 : 256;
        uint64_t rows = t.ne[1] * t.ne[2] * t.ne[3];
        if (t.type == 0) out->bytes = t.ne[0] * rows * 4;
        else if (t.type == 1) out->bytes = t.ne[0] * rows * 2;
        else if (bb && t.ne[0] % per == 0) out->bytes = t.ne[0] / per * bb * rows;
        else return ZMOE_ERR_TYPE;
        if (out->file_offset + out->bytes > g->file_bytes) return ZMOE_ERR_SHAPE;
        return ZMOE_OK;
    }
    return ZMOE_ERR_STATE;   // no such tensor
}

int zmoe_gguf_read(zmoe_gguf *g, const zmoe_gguf_tensor *t, void *dst_host, uint64_t first_byte, uint64_t n_bytes) {
    if (!g || !t || !dst_host || first_byte + n_bytes > t->bytes) return ZMOE_ERR_ARG;
    if (fseek(g->f, (long)(t->file_offset + first_byte), SEEK_SET) != 0) return ZMOE_ERR_ARG;
    return fread(dst_host, 1, n_bytes, g->f) == n_bytes ? ZMOE_OK : ZMOE_ERR_SHAPE;
}

int zmoe_gguf_load_experts(zmoe_gguf *g, int layer, void *gate_dev, void *up_dev, void *down_dev, zmoe_gguf_tensor *info3,
                           void *stream) {
    if (!g || layer < 0 || !gate_dev || !up_dev || !down_dev) return ZMOE_ERR_ARG;
    static const char *kind[3] = {"ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"};
    void *dst[3] = {gate_dev, up_dev, down_dev};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < 3; ++i) {
        char name[96];
        snprintf(name, sizeof(name), "blk.%d.%s.weight", layer, kind[i]);
        zmoe_gguf_tensor t;
        const int rc = zmoe_gguf_find(g, name, &t);
        if (rc) return rc;
        if (t.n_dims != 3) return ZMOE_ERR_SHAPE;     // [row length, rows, experts]
        if (info3) info3[i] = t;
        // through a pinned staging buffer, 64 MiB at a time
        const uint64_t chunk = 64ull << 20;
        void *stage = nullptr;
        if (cudaHostAlloc(&stage, (size_t)(t.bytes < chunk ? t.bytes : chunk), cudaHostAllocDefault) != cudaSuccess)
            return ZMOE_ERR_CUDA;
        int err = 0;
        for (uint64_t off = 0; off < t.bytes && !err; off += chunk) {
            const uint64_t n = t.bytes - off < chunk ? t.bytes - off : chunk;
            err = zmoe_gguf_read(g, &t, stage, off, n);
            if (!err && cudaMemcpyAsync(static_cast<uint8_t *>(dst[i]) + off, stage, (size_t)n, cudaMemcpyHostToDevice, st) != cudaSuccess)
                err = ZMOE_ERR_CUDA;
            if (!err && cudaStreamSynchronize(st) != cudaSuccess) err = ZMOE_ERR_CUDA;   // the staging buffer is reused
        }
        cudaFreeHost(stage);
        if (err) return err;
    }
    return ZMOE_OK;
}

}  // extern "C"
