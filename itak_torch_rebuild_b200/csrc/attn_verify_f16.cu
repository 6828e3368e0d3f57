// Multi-row causal GQA attention over the f16 resident cache: the speculative
// verify block (a handful of rows appended, then attended together) and short
// prefill chunks.
//
// Stands in for gqa_attention with several queries
// (crates/attention/src/attention.rs:160-213), called after all rows of the
// block were appended (crates/arch-llama/src/model.rs:212-228), and for the
// reference's staged flash kernel over f16 KV
// (crates/wgpu-compute/src/kernels/k6_attention.rs:429-592, 642-914): row r of
// the block sits at position q_pos0 + r and sees keys kp <= its position (and
// kp > position - window on a sliding layer).
//
// Here the work really is a small dense contraction: M = rows x heads of the
// GQA group.  A (query row, head) pair takes two rows of an m16 tensor-core
// tile - the hi and lo f16 terms of its f32 query / softmax weights - so one
// warp owns 8 pairs and a CTA of 4 warps owns 32 pairs (7 rows x 4 heads = 28
// in the speculative configuration).  All warps consume the same 64-key K/V
// tiles, staged once per CTA by a 3-deep cp.async pipeline into XOR-swizzled
// shared memory; the key range is split across CTAs exactly as in the decode
// kernel, with the last-arriving CTA merging the partials.
//
// Bound: HBM (the block's K/V stream); the tensor pipe runs 4x the decode
// kernel's work per byte and stays far from its limit.
#include "attn_common.cuh"

namespace itk {

namespace {

constexpr int kVerThreads = 128;  // 4 warps
constexpr int kVerTile = 64;     // keys per tile
constexpr int kPairsPerCta = 32; // (row, head) pairs per CTA: 8 per warp
constexpr int kVerStages = 3;

template <int D>
__global__ void __launch_bounds__(kVerThreads, 2) verify_f16_kernel(const __grid_constant__ AttnLaunch p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kRowBytes = D * 2;
    constexpr int kTileBytes = kVerTile * kRowBytes;  // K (or V) tile
    constexpr int kChunksPerRow = D / 8;
    constexpr int KS = D / 16;
    constexpr int NT = D / 8;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t split = blockIdx.x, seq = blockIdx.z;
    const uint32_t pchunks = (p.rows * min(p.group, static_cast<uint32_t>(kHeadsPerCta)) + kPairsPerCta - 1) / kPairsPerCta;
    const uint32_t hy = blockIdx.y / pchunks, pc = blockIdx.y % pchunks;
    const SeqDesc sd = p.seq[seq];
    const uint32_t kvh = hy / p.gchunks, gc = hy % p.gchunks;
    const uint32_t head0 = kvh * p.group + gc * kHeadsPerCta;
    const uint32_t nh = min(static_cast<uint32_t>(kHeadsPerCta), p.group - gc * kHeadsPerCta);
    const uint32_t n_pairs = p.rows * nh;
    const uint32_t ring = p.layer.ring;
    const uint32_t window = p.layer.window;

    // This CTA's slice [k0, k1) of the positions [kv_lo, kv_hi) the block can see.
    const uint32_t n = sd.kv_hi - sd.kv_lo;
    uint32_t chunk = (n + p.splits - 1) / p.splits;
    chunk = (chunk + kVerTile - 1) / kVerTile * kVerTile;
    const uint32_t k0 = min(n, split * chunk);
    const uint32_t k1 = min(n, k0 + chunk);
    const uint32_t span = k1 - k0;
    const uint32_t ntiles = (span + kVerTile - 1) / kVerTile;
    const uint32_t s0 = (sd.kv_lo + k0) % ring;

    const size_t stream = (static_cast<size_t>(sd.slot) * p.layer.kv_heads + kvh) * ring * D;
    const __half* kbase = static_cast<const __half*>(p.layer.k) + stream;
    const __half* vbase = static_cast<const __half*>(p.layer.v) + stream;

    // This thread's pair: row g of the warp's m16 tile (hi) and row g + 8 (lo).
    const uint32_t pair = pc * kPairsPerCta + warp * 8 + g;
    const bool live = pair < n_pairs;
    const uint32_t prow = live ? pair / nh : 0, phead = live ? pair % nh : 0;
    // Visible positions of the pair's row, relative to kv_lo + k0: [vis_lo, vis_hi).
    const uint32_t ppos = sd.q_pos0 + prow;
    uint32_t abs_lo = sd.kv_lo;
    if (window != 0 && ppos + 1 > window) abs_lo = max(abs_lo, ppos + 1 - window);
    const int64_t rel0 = static_cast<int64_t>(sd.kv_lo) + k0;
    const int64_t vis_lo = live ? static_cast<int64_t>(abs_lo) - rel0 : 0;
    const int64_t vis_hi = live ? static_cast<int64_t>(ppos) + 1 - rel0 : 0;

    uint32_t qa[KS][4];
    {
        const float* qrow = p.q + ((static_cast<size_t>(seq) * p.rows + prow) * p.q_heads + head0 + phead) * D;
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
    auto load_tile = [&](uint32_t tile) {
        const uint32_t stage = tile % kVerStages;
        const uint32_t kbuf = smem_base + stage * 2 * kTileBytes, vbuf = kbuf + kTileBytes;
        const uint32_t row0 = tile * kVerTile;
#pragma unroll
        for (int i = 0; i < kVerTile * kChunksPerRow / kVerThreads; ++i) {
            const int cid = i * kVerThreads + tid;
            const int row = cid / kChunksPerRow, c = cid % kChunksPerRow;
            const uint32_t kr = row0 + row;
            const bool valid = kr < span;
            uint32_t srow = s0 + kr;
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
    for (int s = 0; s < kVerStages - 1; ++s) {
        if (static_cast<uint32_t>(s) < ntiles) load_tile(s);
        cp_async_commit();
    }

    const int mi = lane >> 3, rr = lane & 7;
    for (uint32_t tile = 0; tile < ntiles; ++tile) {
        cp_async_wait<kVerStages - 2>();
        __syncthreads();  // tile landed for every thread; everyone is done with the stage refilled below
        if (tile + kVerStages - 1 < ntiles) load_tile(tile + kVerStages - 1);
        cp_async_commit();

        const uint32_t stage = tile % kVerStages;
        const uint32_t kbuf = smem_base + stage * 2 * kTileBytes, vbuf = kbuf + kTileBytes;
        const uint32_t row0 = tile * kVerTile;

        // S(16 x 64 keys) = Q(16 x D) * K^T
        float s[kVerTile / 8][4];
#pragma unroll
        for (int j = 0; j < kVerTile / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int jn = 0; jn < kVerTile / 16; ++jn) {
            const int krow = 16 * jn + ((mi >> 1) << 3) + rr;
            const uint32_t rbase = kbuf + krow * kRowBytes;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, rbase + (((2 * ks + (mi & 1)) ^ rr) << 4));
                mma_16816(s[2 * jn], qa[ks], b[0], b[1]);
                mma_16816(s[2 * jn + 1], qa[ks], b[2], b[3]);
            }
        }
        // hi + lo, scale, per-row causal / window mask, online softmax for this thread's pair
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < kVerTile / 8; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int64_t kr = static_cast<int64_t>(row0) + 8 * j + 2 * t + e;
                float v = (s[j][e] + s[j][e + 2]) * sl;
                v = (kr >= vis_lo && kr < vis_hi) ? v : -INFINITY;
                s[j][e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // nothing visible yet: weights stay zero
        const float corr = fast_exp2(m - m_use);
        m = m_new;
        l *= corr;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            o[i][0] *= corr;
            o[i][1] *= corr;
            o[i][2] *= corr;
            o[i][3] *= corr;
        }
        // O(16 x D) += P(16 x 64 keys) * V(64 keys x D), 16 keys at a time
#pragma unroll
        for (int kg = 0; kg < kVerTile / 16; ++kg) {
            uint32_t pa[4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float p0 = fast_exp2(s[2 * kg + j][0] - m_use), p1 = fast_exp2(s[2 * kg + j][1] - m_use);
                l += p0 + p1;
                __half h0, l0, h1, l1;
                split_half(p0, h0, l0);
                split_half(p1, h1, l1);
                pa[2 * j] = pack_half2(h0, h1);
                pa[2 * j + 1] = pack_half2(l0, l1);
            }
            const int vrow = 16 * kg + ((mi & 1) << 3) + rr;
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

    // Each warp owns its own pairs: no cross-warp merge.  l is a per-thread partial sum over the quad.
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    __shared__ int s_flag;
    const uint32_t HYP = p.layer.kv_heads * p.gchunks * pchunks;
    const size_t cell = static_cast<size_t>(seq) * HYP + blockIdx.y;
    float* out_row = p.out + ((static_cast<size_t>(seq) * p.rows + prow) * p.q_heads + head0 + phead) * D;
    if (p.splits == 1) {
        if (live) {
            const float inv = 1.f / l;
#pragma unroll
            for (int i = 0; i < NT; ++i)
                *reinterpret_cast<float2*>(out_row + 8 * i + 2 * t) =
                    make_float2((o[i][0] + o[i][2]) * inv, (o[i][1] + o[i][3]) * inv);
        }
        return;
    }
    const uint32_t lp = warp * 8 + g;  // pair index inside the CTA
    float* po = p.part_o + ((cell * p.splits + split) * kPairsPerCta + lp) * D;
    float* pml = p.part_ml + ((cell * p.splits + split) * kPairsPerCta + lp) * 2;
    if (live) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
            *reinterpret_cast<float2*>(po + 8 * i + 2 * t) = make_float2(o[i][0] + o[i][2], o[i][1] + o[i][3]);
        if (t == 0) {
            pml[0] = m;
            pml[1] = l;
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(p.tickets + cell, 1u);
        s_flag = (ticket == p.splits - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_flag == 0) return;
    __threadfence();
    // The last CTA merges every split for the cell's pairs.
    const float* all_o = p.part_o + cell * p.splits * kPairsPerCta * D;
    const float* all_ml = p.part_ml + cell * p.splits * kPairsPerCta * 2;
    const uint32_t cta_pairs = min(static_cast<uint32_t>(kPairsPerCta), n_pairs - pc * kPairsPerCta);
    constexpr uint32_t kSmemBytes = kVerStages * 2 * kTileBytes;
    if (p.splits * kPairsPerCta * 12u <= kSmemBytes) {
        // Every split's (max, sum) pairs come into shared memory in one round trip (the tile stages are idle), the
        // splits' weights per pair follow from them, and every output is a weighted sum over the splits with all of a
        // thread's loads of one split (two, at head_dim 64) in flight - not one dependent round trip per split and output.
        float* w_s = reinterpret_cast<float*>(smem);                               // [splits][32]
        float2* ml_s = reinterpret_cast<float2*>(w_s + p.splits * kPairsPerCta);  // [splits][32]
        const float2* ml2 = reinterpret_cast<const float2*>(all_ml);
        for (uint32_t i = tid; i < p.splits * kPairsPerCta; i += kVerThreads) ml_s[i] = __ldcg(ml2 + i);
        __syncthreads();
        if (static_cast<uint32_t>(tid) < cta_pairs) {
            float M = -INFINITY;
            for (uint32_t s = 0; s < p.splits; ++s) M = fmaxf(M, ml_s[s * kPairsPerCta + tid].x);
            float L = 0.f;
            for (uint32_t s = 0; s < p.splits; ++s) {
                const float2 ml = ml_s[s * kPairsPerCta + tid];
                const float w = (ml.x == -INFINITY) ? 0.f : fast_exp2(ml.x - M);
                w_s[s * kPairsPerCta + tid] = w;
                L += w * ml.y;
            }
            const float inv = 1.f / L;
            for (uint32_t s = 0; s < p.splits; ++s) w_s[s * kPairsPerCta + tid] *= inv;
        }
        __syncthreads();
        constexpr int kOut = kPairsPerCta * D / kVerThreads;  // outputs per thread: 16 or 32
        constexpr int kBatch = kOut <= 16 ? 2 : 1;  // (kept small: the epilogue must not raise the kernel's register count)
        float acc[kOut];
#pragma unroll
        for (int i = 0; i < kOut; ++i) acc[i] = 0.f;
        for (uint32_t s0 = 0; s0 < p.splits; s0 += kBatch) {
            float v[kBatch][kOut];
#pragma unroll
            for (int bb = 0; bb < kBatch; ++bb) {
                const uint32_t s = min(s0 + bb, p.splits - 1);  // a repeated split past the end weighs zero
                const float* src = all_o + static_cast<size_t>(s) * kPairsPerCta * D;
#pragma unroll
                for (int i = 0; i < kOut; ++i) {
                    const uint32_t idx = tid + i * kVerThreads;
                    v[bb][i] = idx < cta_pairs * D ? __ldcg(src + idx) : 0.f;
                }
            }
#pragma unroll
            for (int bb = 0; bb < kBatch; ++bb) {
                const bool real = s0 + bb < p.splits;
#pragma unroll
                for (int i = 0; i < kOut; ++i) {
                    const uint32_t idx = tid + i * kVerThreads;
                    acc[i] += ((real && idx < cta_pairs * D) ? w_s[(s0 + bb) * kPairsPerCta + idx / D] : 0.f) * v[bb][i];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kOut; ++i) {
            const uint32_t idx = tid + i * kVerThreads;
            if (idx < cta_pairs * D) {
                const uint32_t gp = pc * kPairsPerCta + idx / D;
                p.out[((static_cast<size_t>(seq) * p.rows + gp / nh) * p.q_heads + head0 + gp % nh) * D + idx % D] = acc[i];
            }
        }
    } else {
        for (uint32_t idx = tid; idx < cta_pairs * D; idx += kVerThreads) {
            const uint32_t q = idx / D, dd = idx % D;
            float M = -INFINITY, L = 0.f, O = 0.f;
            for (uint32_t s = 0; s < p.splits; ++s) {
                const float ms = __ldcg(all_ml + (static_cast<size_t>(s) * kPairsPerCta + q) * 2);
                if (ms == -INFINITY) continue;
                const float ls = __ldcg(all_ml + (static_cast<size_t>(s) * kPairsPerCta + q) * 2 + 1);
                const float os = __ldcg(all_o + (static_cast<size_t>(s) * kPairsPerCta + q) * D + dd);
                const float Mn = fmaxf(M, ms);
                const float a = fast_exp2(M - Mn);
                const float b = fast_exp2(ms - Mn);
                O = O * a + os * b;
                L = L * a + ls * b;
                M = Mn;
            }
            const uint32_t gp = pc * kPairsPerCta + q;
            const uint32_t r = gp / nh, h = gp % nh;
            p.out[((static_cast<size_t>(seq) * p.rows + r) * p.q_heads + head0 + h) * D + dd] = O / L;
        }
    }
    if (tid == 0) p.tickets[cell] = 0u;
}

template <int D>
constexpr size_t verify_smem_bytes() {
    return static_cast<size_t>(kVerStages) * 2 * kVerTile * D * 2;
}

}  // namespace

bool verify_f16_supported(uint32_t head_dim, uint32_t rows, uint32_t group) {
    (void)group;
    return rows >= 2 && rows <= 64 && (head_dim == 128 || head_dim == 64);
}

uint32_t verify_pair_chunks(uint32_t rows, uint32_t group) {
    const uint32_t nh = group < static_cast<uint32_t>(kHeadsPerCta) ? group : kHeadsPerCta;
    return (rows * nh + kPairsPerCta - 1) / kPairsPerCta;
}

cudaError_t configure_verify_f16() {
    cudaError_t e = cudaFuncSetAttribute(verify_f16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(verify_smem_bytes<128>()));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(verify_f16_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(verify_smem_bytes<64>()));
}

cudaError_t launch_verify_f16(const AttnLaunch& p, cudaStream_t s, uint64_t* launches) {
    const uint32_t pchunks = verify_pair_chunks(p.rows, p.group);
    const dim3 grid(p.splits, p.layer.kv_heads * p.gchunks * pchunks, p.n_seqs);
    if (p.layer.head_dim == 128)
        verify_f16_kernel<128><<<grid, kVerThreads, verify_smem_bytes<128>(), s>>>(p);
    else if (p.layer.head_dim == 64)
        verify_f16_kernel<64><<<grid, kVerThreads, verify_smem_bytes<64>(), s>>>(p);
    else
        return cudaErrorInvalidValue;
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk
