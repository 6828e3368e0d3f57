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
