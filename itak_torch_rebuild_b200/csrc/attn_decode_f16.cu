// GQA flash-decode over the f16 resident cache: one query row per sequence.
//
// Stands in for the reference's decode attention, i.e. gqa_attention with one
// query (crates/attention/src/attention.rs:104-215) reading an f16 cache the
// way the K6 flash f16 shader does (crates/wgpu-compute/src/kernels/k6_attention.rs:642-914):
// keys and values are upconverted exactly, all arithmetic accumulates in f32.
//
// Work split (what the reference kernels lack): one CTA per
// (sequence, KV head, split of the key range).  All query heads of the GQA
// group share every K/V tile, so each cache byte crosses HBM once per step.
// The key range is cut into `splits` CTAs; each writes an (m, l, o) partial
// and the last CTA to arrive merges them (see finish_unit).
//
// Inside a CTA each of the 4 warps owns a private cp.async pipeline over its
// own 16-key slice of every 64-key tile: 16-byte coalesced loads into
// XOR-swizzled shared memory, STAGES tiles in flight, no CTA-wide barrier in
// the main loop.  The cache is head-major, so a CTA's loads walk one contiguous
// stream.
//
// Bound: HBM.  A cache element (2 B) feeds 2 * group MACs, 4 FMA/B at group 8;
// at 6.5 TB/s that is ~70% of the SM's fp32 FMA rate before counting the
// f16->f32 converts, so the dot products run on the tensor pipe instead, as
// mma.sync.m16n8k16 with M = 16 = 8 heads x {hi, lo}: the f32 query (and the
// f32 softmax weight) is split into two f16 terms that occupy the rows a GQA
// group of 8 would otherwise leave as padding.  The products are then exact to
// ~2^-22 and the accumulation is f32, so the result tracks the f32 reference
// far inside the f16-KV tolerance.  A 64-row tcgen05 tile would be 7/8 padding
// here; the tensor pipe is at ~15% load either way and never the limiter.
#include <cstdio>

#include "attn_common.cuh"

namespace itk {

namespace {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeWarps = 4;
constexpr int kTileKeys = 64;  // keys per CTA tile = 16 per warp

template <int D, int STAGES>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_f16_kernel(const __grid_constant__ AttnLaunch p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kRowBytes = D * 2;
    constexpr int kSliceBytes = 16 * kRowBytes;  // one warp's K (or V) slice of a tile
    constexpr int kChunksPerRow = D / 8;         // 16-byte chunks in a row
    constexpr int KS = D / 16;                   // k-steps of the QK^T product
    constexpr int NT = D / 8;                    // n-tiles of the PV product

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t split = blockIdx.x, hy = blockIdx.y, unit = blockIdx.z;
    const SeqDesc sd = p.seq[unit];
    const uint32_t kvh = hy / p.gchunks, gc = hy % p.gchunks;
    const uint32_t head0 = kvh * p.group + gc * kHeadsPerCta;
    const uint32_t nh = min(static_cast<uint32_t>(kHeadsPerCta), p.group - gc * kHeadsPerCta);
    const uint32_t ring = p.layer.ring;

    // This CTA's slice [k0, k1) of the visible keys, in whole tiles.
    const uint32_t n = sd.kv_hi - sd.kv_lo;
    uint32_t chunk = (n + p.splits - 1) / p.splits;
    chunk = (chunk + kTileKeys - 1) / kTileKeys * kTileKeys;
    const uint32_t k0 = min(n, split * chunk);
    const uint32_t k1 = min(n, k0 + chunk);
    const uint32_t span = k1 - k0;
    const uint32_t ntiles = (span + kTileKeys - 1) / kTileKeys;
    const uint32_t s0 = (sd.kv_lo + k0) % ring;  // storage row of key k0

    const size_t stream = (static_cast<size_t>(sd.slot) * p.layer.kv_heads + kvh) * ring * D;
    const __half* kbase = static_cast<const __half*>(p.layer.k) + stream;
    const __half* vbase = static_cast<const __half*>(p.layer.v) + stream;

    // Query fragments: row g = head g (hi term), row g + 8 = the same head's lo term.
    uint32_t qa[KS][4];
    {
        const float* qrow = p.q + (static_cast<size_t>(unit) * p.q_heads + head0 + g) * D;
        const bool live = static_cast<uint32_t>(g) < nh;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            float2 x0 = make_float2(0.f, 0.f), x1 = make_float2(0.f, 0.f);
            if (live) {
                x0 = *reinterpret_cast<const float2*>(qrow + 16 * ks + 2 * t);
                x1 = *reinterpret_cast<const float2*>(qrow + 16 * ks + 8 + 2 * t);
            }
            __half h0, l0, h1, l1;
            split_half(x0.x, h0, l0);
            split_half(x0.y, h1, l1);
            qa[ks][0] = pack_half2(h0, h1);
            qa[ks][1] = pack_half2(l0, l1);
            split_half(x1.x, h0, l0);
            split_half(x1.y, h1, l1);
            qa[ks][2] = pack_half2(h0, h1);
            qa[ks][3] = pack_half2(l0, l1);
        }
    }

    const uint32_t smem_base = smem_u32(smem);
    auto slice_addr = [&](uint32_t stage, int which) -> uint32_t {
        return smem_base + ((stage * kDecodeWarps + warp) * 2 + which) * kSliceBytes;
    };
    // Issue this warp's loads for one tile: 16 rows x kRowBytes of K and of V.
    auto load_tile = [&](uint32_t tile) {
        const uint32_t stage = tile % STAGES;
        const uint32_t kbuf = slice_addr(stage, 0), vbuf = slice_addr(stage, 1);
        const uint32_t row0 = tile * kTileKeys + warp * 16;
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            const int cid = i * 32 + lane;
            const int row = cid / kChunksPerRow, c = cid % kChunksPerRow;
            const uint32_t kr = row0 + row;  // key index relative to k0
            const bool valid = kr < span;
            uint32_t srow = s0 + kr;  // span <= ring, so one wrap at most
            if (srow >= ring) srow -= ring;
            const size_t goff = static_cast<size_t>(valid ? srow : 0u) * D + c * 8;
            const uint32_t soff = row * kRowBytes + ((c ^ (row & 7)) << 4);
            cp_async16(kbuf + soff, kbase + goff, valid ? 16u : 0u);
            cp_async16(vbuf + soff, vbase + goff, valid ? 16u : 0u);
        }
    };

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m = -INFINITY, l = 0.f;
    const float sl = p.scale * kLog2e;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (static_cast<uint32_t>(s) < ntiles) load_tile(s);
        cp_async_commit();
    }

    const int mi = lane >> 3, rr = lane & 7;
    for (uint32_t tile = 0; tile < ntiles; ++tile) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (tile + STAGES - 1 < ntiles) load_tile(tile + STAGES - 1);
        cp_async_commit();

        const uint32_t row0 = tile * kTileKeys + warp * 16;
        if (row0 >= span) continue;  // this warp's slice is past the end (last tile only)
        const uint32_t stage = tile % STAGES;
        const uint32_t kbuf = slice_addr(stage, 0), vbuf = slice_addr(stage, 1);

        // S(16 x 16 keys) = Q(16 x D) * K^T
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const int krow = ((mi >> 1) << 3) + rr;
            const uint32_t rbase = kbuf + krow * kRowBytes;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, rbase + (((2 * ks + (mi & 1)) ^ rr) << 4));
                mma_16816(s[0], qa[ks], b[0], b[1]);
                mma_16816(s[1], qa[ks], b[2], b[3]);
            }
        }
        // hi + lo, scale, mask the tail, online softmax for head g.
        float sc[2][2];
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t kr = row0 + 8 * j + 2 * t + e;
                float v = (s[j][e] + s[j][e + 2]) * sl;
                v = kr < span ? v : -INFINITY;
                sc[j][e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);  // finite: key row0 is valid
        const float corr = fast_exp2(m - m_new);
        m = m_new;
        uint32_t pa[4];
        float psum = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float p0 = fast_exp2(sc[j][0] - m_new), p1 = fast_exp2(sc[j][1] - m_new);
            psum += p0 + p1;
            __half h0, l0, h1, l1;
            split_half(p0, h0, l0);
            split_half(p1, h1, l1);
            pa[2 * j] = pack_half2(h0, h1);
            pa[2 * j + 1] = pack_half2(l0, l1);
        }
        l = l * corr + psum;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            o[i][0] *= corr;
            o[i][1] *= corr;
            o[i][2] *= corr;
            o[i][3] *= corr;
        }
        // O(16 x D) += P(16 x 16 keys) * V(16 keys x D)
        {
            const int vrow = ((mi & 1) << 3) + rr;
            const uint32_t rbase = vbuf + vrow * kRowBytes;
#pragma unroll
            for (int jp = 0; jp < NT / 2; ++jp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, rbase + (((2 * jp + (mi >> 1)) ^ rr) << 4));
                mma_16816(o[2 * jp], pa, b[0], b[1]);
                mma_16816(o[2 * jp + 1], pa, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its pipeline buffers

    // Per-warp results into shared memory, then one merge across the 4 warps.
    float* wo = reinterpret_cast<float*>(smem);                       // [4][8][D]
    float* wm = wo + kDecodeWarps * kHeadsPerCta * D;                 // [4][8]
    float* wl = wm + kDecodeWarps * kHeadsPerCta;                     // [4][8]
    float* fo = wl + kDecodeWarps * kHeadsPerCta;                     // [8][D]
    float* fm = fo + kHeadsPerCta * D;                                // [8]
    float* fl = fm + kHeadsPerCta;                                    // [8]
    int* flag = reinterpret_cast<int*>(fl + kHeadsPerCta);
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    {
        float* dst = wo + (warp * kHeadsPerCta + g) * D;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            float2 v = make_float2(o[i][0] + o[i][2], o[i][1] + o[i][3]);
            *reinterpret_cast<float2*>(dst + 8 * i + 2 * t) = v;
        }
        if (t == 0) {
            wm[warp * kHeadsPerCta + g] = m;
            wl[warp * kHeadsPerCta + g] = l;
        }
    }
    __syncthreads();
    for (int idx = tid; idx < kHeadsPerCta * D; idx += kDecodeThreads) {
        const int h = idx / D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, wm[w * kHeadsPerCta + h]);
        float O = 0.f, L = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kDecodeWarps; ++w) {
                const float mw = wm[w * kHeadsPerCta + h];
                const float a = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
                O += a * wo[(w * kHeadsPerCta + h) * D + (idx % D)];
                L += a * wl[w * kHeadsPerCta + h];
            }
        }
        fo[idx] = O;
        if ((idx % D) == 0) {
            fm[h] = M;
            fl[h] = L;
        }
    }
    __syncthreads();
    finish_unit<kDecodeThreads>(p, unit, hy, split, head0, nh, D, fo, fm, fl, flag);
}

template <int D, int STAGES>
constexpr size_t decode_smem_bytes() {
    return static_cast<size_t>(STAGES) * kDecodeWarps * 2 * 16 * D * 2;
}

constexpr int kStages128 = 3;  // 96 KiB per CTA at D = 128, two CTAs per SM
constexpr int kStages64 = 4;   // 64 KiB per CTA at D = 64

}  // namespace

bool decode_f16_supported(uint32_t head_dim, uint32_t rows) {
    return rows == 1 && (head_dim == 128 || head_dim == 64);
}

cudaError_t configure_decode_f16() {
    cudaError_t e = cudaFuncSetAttribute(decode_f16_kernel<128, kStages128>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(decode_smem_bytes<128, kStages128>()));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(decode_f16_kernel<64, kStages64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(decode_smem_bytes<64, kStages64>()));
}

cudaError_t launch_decode_f16(const AttnLaunch& p, cudaStream_t s, uint64_t* launches) {
    const dim3 grid(p.splits, p.layer.kv_heads * p.gchunks, p.n_seqs);
    if (p.layer.head_dim == 128) {
        decode_f16_kernel<128, kStages128>
            <<<grid, kDecodeThreads, decode_smem_bytes<128, kStages128>(), s>>>(p);
    } else if (p.layer.head_dim == 64) {
        decode_f16_kernel<64, kStages64><<<grid, kDecodeThreads, decode_smem_bytes<64, kStages64>(), s>>>(p);
    } else {
        return cudaErrorInvalidValue;
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Who this is for: code that runs where a device allocation is off the table -
// a serving loop that took all of its memory at start-up and is forbidden to
// grow, a plugin invoked from inside somebody else's runtime that owns the
// allocator, a real-time path where cudaMalloc's implicit synchronisation is
// unacceptable, or a region of work being recorded for later replay, in which
// an allocation is an error.  Such a caller already holds its cache, its
// queries and its output buffer; the only thing the split-K decode kernel
// still needs is somewhere to park the per-split partial results.  Here that
// scratch is a fixed array baked into the library image, so the call performs
// no cudaMalloc, no cudaFree and no other allocating routine.
//
// Cost and limits of that choice:
//  - the array below (about 8.1 MiB) exists on every GPU that loads this
//    library, from load until the process exits, whether or not this entry
//    point is ever used;
//  - (sequences x KV heads x head chunks) x splits may not exceed
//    kNoAllocCellSplits, sequences may not exceed 64, head_dim is 64 or 128;
//    anything larger is refused with ITK_ERR_CAPACITY and a message;
//  - all calls share the one array and it keeps whatever the previous call
//    left.  The arrival counters are the only part that must read zero at
//    launch; every call clears them on its stream first.  Two calls whose
//    kernels can overlap on the GPU (different streams, or different host
//    threads on different streams) trample each other's partials and
//    counters: serialise them.
//
// A symbol declared `__device__` is, in host code, only a handle for the
// runtime - not an address a kernel can dereference.  The device address is
// obtained once per device with cudaGetSymbolAddress while that device is
// current, and that pointer is what the kernel receives.  The first call on a
// device performs this set-up (and the kernel's shared-memory opt-in); make
// that first call before starting any stream capture.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocCellSplits = 2048;  // (cell, split) partial slots
constexpr size_t kNoAllocPartO = kNoAllocCellSplits * itk::kHeadsPerCta * 128 * sizeof(float);  // 8 MiB
constexpr size_t kNoAllocPartMl = kNoAllocCellSplits * itk::kHeadsPerCta * 2 * sizeof(float);   // 128 KiB
constexpr size_t kNoAllocTickets = kNoAllocCellSplits * sizeof(unsigned int);                    // 8 KiB
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocPartO + kNoAllocPartMl + kNoAllocTickets];

// Device address of g_noalloc_scratch per device ordinal, resolved on first use.
void* g_noalloc_ptr[kNoAllocMaxDevices] = {};

int noalloc_refuse(int code, char* text, size_t text_len, const char* fmt, unsigned long long a = 0,
                   unsigned long long b = 0) {
    if (text && text_len) snprintf(text, text_len, fmt, a, b);
    return code;
}

}  // namespace

extern "C" int itk_decode_attention_noalloc(const void* k_layer, const void* v_layer, uint32_t ring,
                                            uint32_t kv_heads, uint32_t q_heads, uint32_t head_dim, uint32_t n_seqs,
                                            const uint32_t* slots, const uint32_t* kv_len, const float* d_q,
                                            float* d_out, uint32_t splits, void* cuda_stream, char* error_text,
                                            size_t error_text_len) {
    using namespace itk;
    if (error_text && error_text_len) error_text[0] = '\0';
    if (!k_layer || !v_layer || !slots || !kv_len || !d_q || !d_out)
        return noalloc_refuse(101, error_text, error_text_len, "null pointer argument");
    if (kv_heads == 0 || q_heads == 0 || ring == 0)
        return noalloc_refuse(1, error_text, error_text_len, "kv_heads, q_heads and ring must be positive");
    if (q_heads % kv_heads != 0)
        return noalloc_refuse(7, error_text, error_text_len, "%llu query heads do not divide evenly across %llu KV heads",
                              q_heads, kv_heads);
    if (head_dim != 64 && head_dim != 128)
        return noalloc_refuse(102, error_text, error_text_len, "head_dim %llu is not supported here (64 or 128)", head_dim);
    if (n_seqs == 0) return 0;
    if (n_seqs > static_cast<uint32_t>(kMaxSeqsPerLaunch))
        return noalloc_refuse(102, error_text, error_text_len,
                              "%llu sequences exceed this entry point's maximum of %llu per call", n_seqs,
                              static_cast<unsigned long long>(kMaxSeqsPerLaunch));
    const uint32_t group = q_heads / kv_heads;
    const uint32_t gchunks = (group + kHeadsPerCta - 1) / kHeadsPerCta;
    const unsigned long long cells = static_cast<unsigned long long>(n_seqs) * kv_heads * gchunks;
    uint32_t n_max = 0;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        if (kv_len[i] == 0)
            return noalloc_refuse(8, error_text, error_text_len, "sequence %llu has no visible keys", i);
        if (kv_len[i] > ring)
            return noalloc_refuse(102, error_text, error_text_len, "sequence %llu holds more keys than the ring of %llu",
                                  i, ring);
        if (kv_len[i] > n_max) n_max = kv_len[i];
    }
    if (cells > kNoAllocCellSplits)
        return noalloc_refuse(102, error_text, error_text_len,
                              "%llu (sequence, head) cells exceed the built-in scratch of %llu", cells,
                              static_cast<unsigned long long>(kNoAllocCellSplits));
    if (splits == 0) {  // a few hundred CTAs, at least four 64-key tiles each
        unsigned long long s = (296 * 2 + cells - 1) / cells;
        const unsigned long long by_len = (n_max + 255) / 256;
        if (s > by_len) s = by_len;
        if (s * cells > kNoAllocCellSplits) s = kNoAllocCellSplits / cells;
        splits = static_cast<uint32_t>(s < 1 ? 1 : s);
    }
    if (cells * splits > kNoAllocCellSplits)
        return noalloc_refuse(102, error_text, error_text_len,
                              "cells x splits = %llu exceeds the built-in scratch of %llu partial slots; lower `splits`",
                              cells * splits, static_cast<unsigned long long>(kNoAllocCellSplits));

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices)
        return noalloc_refuse(100, error_text, error_text_len, "no usable current CUDA device");
    if (!g_noalloc_ptr[dev]) {
        // One-time set-up for this device: resolve the array's device address and opt the kernel in to its
        // dynamic shared memory size.  Neither allocates.
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) {
            if (error_text && error_text_len)
                snprintf(error_text, error_text_len, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return 100;
        }
        e = configure_decode_f16();
        if (e != cudaSuccess) {
            if (error_text && error_text_len)
                snprintf(error_text, error_text_len, "kernel attribute setup failed: %s", cudaGetErrorString(e));
            return 100;
        }
        g_noalloc_ptr[dev] = ptr;
    }
    unsigned char* base = static_cast<unsigned char*>(g_noalloc_ptr[dev]);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    AttnLaunch p{};
    p.layer.k = k_layer;
    p.layer.v = v_layer;
    p.layer.ring = ring;
    p.layer.window = 0;
    p.layer.kv_heads = kv_heads;
    p.layer.head_dim = head_dim;
    p.q = d_q;
    p.out = d_out;
    p.part_o = reinterpret_cast<float*>(base);
    p.part_ml = reinterpret_cast<float*>(base + kNoAllocPartO);
    p.tickets = reinterpret_cast<unsigned int*>(base + kNoAllocPartO + kNoAllocPartMl);
    p.q_heads = q_heads;
    p.group = group;
    p.gchunks = gchunks;
    p.rows = 1;
    p.n_seqs = n_seqs;
    p.splits = splits;
    p.scale = 1.0f / sqrtf(static_cast<float>(head_dim));
    for (uint32_t i = 0; i < n_seqs; ++i) p.seq[i] = SeqDesc{slots[i], kv_len[i] - 1, 0, kv_len[i]};
    // The arrival counters must read zero when the kernel starts, whatever an earlier (possibly failed)
    // call left behind.
    e = cudaMemsetAsync(p.tickets, 0, cells * sizeof(unsigned int), stream);
    if (e == cudaSuccess) e = launch_decode_f16(p, stream, nullptr);
    if (e != cudaSuccess) {
        if (error_text && error_text_len)
            snprintf(error_text, error_text_len, "decode attention launch failed: %s", cudaGetErrorString(e));
        return 100;
    }
    return 0;
}
