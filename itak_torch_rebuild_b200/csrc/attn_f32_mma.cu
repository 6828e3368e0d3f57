// GQA attention over an f32 resident cache on the tensor cores: decode rows,
// speculative blocks and prefill chunks of any length, head_dim 64 or 128.
//
// Stands in for gqa_attention (crates/attention/src/attention.rs:104-215) on
// the cache the reference itself keeps (f32 rows, crates/attention/src/cache.rs:11-15):
// the configuration its CPU backend runs (a 512-row prefill, then decode
// steps).  Row r of a block sits at position q_pos0 + r and sees the keys
// kp <= its position (kp > position - window on a sliding layer) that are
// stored.
//
// The contraction runs as tf32 tensor-core products with three terms per
// product (x = hi + lo with hi = tf32(x), lo = x - hi cut to tf32; x*y is
// taken as lo*hi + hi*lo + hi*hi, accumulated in f32), which reproduces the
// f32 product to about 2^-20: inside the 1e-4 tolerance of an f32 cache with
// two orders of magnitude to spare, where a single tf32 product (2^-11) is not.
//
// M = (row, head) pairs of one GQA group, 16 per warp tile.  Two shapes of CTA
// (4 warps):
//   WK = 1  prefill / verify blocks: 64 pairs per CTA, a warp owns 16 pairs
//           and walks every key of the 32-key tile;
//   WK = 4  decode (at most 16 pairs): all four warps own the same 16 pairs
//           and each walks a quarter of the tile's keys; their results are
//           merged through shared memory at the end.
// K/V tiles are staged once per CTA by cp.async into shared memory with a
// row pitch of D + 4 floats (bank-conflict-free for both operand patterns,
// every fragment address a constant away from the thread's base) and split
// into hi/lo terms as the fragments are read.  Small tiles and two stages keep a CTA at
// 51 KiB (head_dim 64) so that four CTAs - sixteen warps - share an SM: the
// warps' chains of conversions and dependent products hide behind each other.
// The key range of a pair block ends at the block's last row (causal bound)
// and starts at its first row's window.  It is cut into parts of one size per
// sequence (the longest block's range over AttnLaunch::splits), so a short
// block has fewer parts than a long one - surplus CTAs leave at once - and
// the last-arriving part of a block merges the others.
//
// Bound: the configuration this serves keeps its whole cache in L2, so a
// launch is bound by latency (decode) or by instruction issue and the tensor
// pipe (prefill: three m16n8k8 products per useful one, operands converted on
// the way in).
#include "attn_common.cuh"

namespace itk {

namespace {

constexpr int kF32Threads = 128;
constexpr int kF32Tile = 32;     // keys per tile
constexpr int kF32Stages = 2;    // K + V tiles in flight: 16 KiB per stage at D 64, 32 KiB at D 128
constexpr int kF32MaxParts = 64; // parts of one block's key range (sizes the merge weights in shared memory)

// x = hi + lo for the three-term product.  hi is x rounded to tf32 (10 mantissa bits) by integer arithmetic on
// the bit pattern - add half a unit of the last kept place, clear the 13 dropped bits: round to nearest, ties away,
// as cvt.rna does, in two instructions (the conversion instruction itself expands to a dozen here).  lo = x - hi is
// exact in f32 and is cut to tf32 width (what the tensor core would read of it anyway): |x - hi - lo| <= 2^-21 |x|.
// An infinity stays an infinity, a NaN a NaN; a finite x within half a tf32 step of the largest f32 becomes an
// infinity, as it does under cvt.rna.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    hi = (__float_as_uint(x) + 0x1000u) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi)) & 0xffffe000u;
}

// D(16x8, f32) += A(16x8, tf32, row) * B(8x8, tf32, col).  With g = lane / 4, t = lane % 4:
//   a[0] = A[g][t]   a[1] = A[g+8][t]   a[2] = A[g][t+4]   a[3] = A[g+8][t+4]
//   b[0] = B[t][g]   b[1] = B[t+4][g]
//   c[0..1] = D[g][2t..2t+1]   c[2..3] = D[g+8][2t..2t+1]
__device__ __forceinline__ void mma_1688(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// the three-term product: small terms first
__device__ __forceinline__ void mma3(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                     const uint32_t (&bh)[2], const uint32_t (&bl)[2]) {
    mma_1688(c, al, bh);
    mma_1688(c, ah, bl);
    mma_1688(c, ah, bh);
}

// One pair block: (sequence, head chunk hy, pair block pc) over part `split` of its key range.
template <int D, int WK>
__device__ __forceinline__ void f32_block(const AttnLaunch& p, unsigned char* smem, uint32_t seq, uint32_t hy, uint32_t pc,
                                          uint32_t pchunks, uint32_t split) {
    constexpr int kStages = kF32Stages;
    constexpr int PB = 4 / WK;                 // pair blocks (of 16) per CTA
    constexpr int PC = 16 * PB;                // pairs per CTA
    constexpr int KW = kF32Tile / WK;          // keys of a tile one warp walks
    constexpr int kChunks = D / 4;             // 16-byte chunks per row
    constexpr int LD = D + 4;                   // row pitch in shared memory, floats (see below)
    constexpr int kTileFloats = kF32Tile * LD;  // one K (or V) tile
    constexpr int KS = D / 8, NT = D / 8;

    // Rows of D floats sit LD = D + 4 floats apart: with a pitch of 4 (mod 32) banks the eight rows x four columns
    // of a K (or Q) fragment read and the four rows x eight columns of a V fragment read both touch 32 different
    // banks, and every fragment address is the thread's base plus a compile-time constant.
    float* q_s = reinterpret_cast<float*>(smem);  // [PC][LD]
    float* tiles = q_s + PC * LD;                 // kStages x (K tile, V tile); the warps' results afterwards
    __shared__ float res_m[4][16], res_l[4][16];
    __shared__ int s_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int pb = warp / WK, ksub = warp % WK;
    const SeqDesc sd = p.seq[seq];
    const uint32_t kvh = hy / p.gchunks, gc = hy % p.gchunks;
    const uint32_t head0 = kvh * p.group + gc * kHeadsPerCta;
    const uint32_t nh = min(static_cast<uint32_t>(kHeadsPerCta), p.group - gc * kHeadsPerCta);
    const uint32_t n_pairs = p.rows * nh;
    const uint32_t ring = p.layer.ring;
    const uint32_t window = p.layer.window;
    const uint32_t first_pair = pc * PC;
    if (first_pair >= n_pairs) return;  // (a chunk of fewer heads than the widest one may need fewer pair blocks)
    const uint32_t cta_pairs = min(static_cast<uint32_t>(PC), n_pairs - first_pair);

    // The positions this pair block can see: from its first row's window to its last row, cut to what is stored.
    const uint32_t first_pos = sd.q_pos0 + first_pair / nh;
    const uint32_t last_pos = sd.q_pos0 + (first_pair + cta_pairs - 1) / nh;
    uint32_t blk_lo = sd.kv_lo;
    if (window != 0 && first_pos + 1 > window) blk_lo = max(blk_lo, first_pos + 1 - window);
    const uint32_t blk_hi = min(sd.kv_hi, last_pos + 1);
    const uint32_t n = blk_hi > blk_lo ? blk_hi - blk_lo : 0u;
    // parts of one size for every block of the sequence: whole tiles, the longest range over p.splits
    const uint32_t seq_tiles = (sd.kv_hi - sd.kv_lo + kF32Tile - 1) / kF32Tile;
    const uint32_t chunk = max(1u, (seq_tiles + p.splits - 1) / p.splits) * kF32Tile;
    const uint32_t parts = max(1u, (n + chunk - 1) / chunk);  // <= p.splits
    if (split >= parts) return;
    const uint32_t k0 = split * chunk;
    const uint32_t k1 = min(n, k0 + chunk);
    const uint32_t span = k1 - k0;
    const uint32_t ntiles = (span + kF32Tile - 1) / kF32Tile;
    const uint32_t s0 = (blk_lo + k0) % ring;

    const size_t stream = (static_cast<size_t>(sd.slot) * p.layer.kv_heads + kvh) * ring * D;
    const float* kbase = static_cast<const float*>(p.layer.k) + stream;
    const float* vbase = static_cast<const float*>(p.layer.v) + stream;

    // A launch that carries the call's new rows (k_new / v_new, f32 [seq][row][kv_heads * D]) reads them from there
    // and stores them itself: an f32 cache holds the rows as they come, so the append is a plain copy, shared out
    // over the pair blocks of the KV head's first head chunk.  The ring slots they take held positions that no row
    // of this call can see (the ring is at least window + chunk rows long).
    const bool fused = p.k_new != nullptr;
    const size_t new_stride = static_cast<size_t>(p.layer.kv_heads) * D;
    const float* knew = fused ? p.k_new + (static_cast<size_t>(seq) * p.rows * p.layer.kv_heads + kvh) * D : nullptr;
    const float* vnew = fused ? p.v_new + (static_cast<size_t>(seq) * p.rows * p.layer.kv_heads + kvh) * D : nullptr;
    if (fused && gc == 0 && split == 0) {
        const uint32_t per = (p.rows + pchunks - 1) / pchunks;
        const uint32_t r0 = min(p.rows, pc * per), r1 = min(p.rows, r0 + per);
        float* kdst = const_cast<float*>(kbase);
        float* vdst = const_cast<float*>(vbase);
        for (uint32_t i = tid; i < (r1 - r0) * kChunks; i += kF32Threads) {
            const uint32_t r = r0 + i / kChunks, c = i % kChunks;
            const uint32_t srow = (sd.q_pos0 + r) % ring;
            const float4 kx = __ldg(reinterpret_cast<const float4*>(knew + r * new_stride) + c);
            const float4 vx = __ldg(reinterpret_cast<const float4*>(vnew + r * new_stride) + c);
            reinterpret_cast<float4*>(kdst + static_cast<size_t>(srow) * D)[c] = kx;
            reinterpret_cast<float4*>(vdst + static_cast<size_t>(srow) * D)[c] = vx;
        }
    }
    // first key row (relative to this part's start) that is one of the call's new rows
    const int64_t new_rel = fused ? static_cast<int64_t>(sd.q_pos0) - (static_cast<int64_t>(blk_lo) + k0) : INT64_MAX;

    const uint32_t smem_tiles = smem_u32(tiles);
    auto load_tile = [&](uint32_t tile) {
        const uint32_t stage = tile % kStages;
        const uint32_t kbuf = smem_tiles + stage * 2 * kTileFloats * 4, vbuf = kbuf + kTileFloats * 4;
        const uint32_t row0 = tile * kF32Tile;
#pragma unroll
        for (int i = 0; i < kF32Tile * kChunks / kF32Threads; ++i) {
            const int cid = i * kF32Threads + tid;
            const int row = cid / kChunks, c = cid % kChunks;
            const uint32_t kr = row0 + row;
            const bool valid = kr < span;
            uint32_t srow = s0 + kr;
            if (srow >= ring) srow -= ring;
            const float* ksrc = kbase + static_cast<size_t>(valid ? srow : 0u) * D + c * 4;
            const float* vsrc = vbase + static_cast<size_t>(valid ? srow : 0u) * D + c * 4;
            if (valid && static_cast<int64_t>(kr) >= new_rel) {
                const size_t noff = static_cast<size_t>(static_cast<int64_t>(kr) - new_rel) * new_stride + c * 4;
                ksrc = knew + noff;
                vsrc = vnew + noff;
            }
            cp_async16(kbuf + row * (LD * 4) + (c << 4), ksrc, valid ? 16u : 0u);
            cp_async16(vbuf + row * (LD * 4) + (c << 4), vsrc, valid ? 16u : 0u);
        }
    };
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (static_cast<uint32_t>(s) < ntiles) load_tile(s);
        cp_async_commit();
    }

    // The block's query rows, pitched like a K tile (dead pairs read as zero).
    for (uint32_t i = tid; i < PC * kChunks; i += kF32Threads) {
        const uint32_t q = i / kChunks, c = i % kChunks;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q < cta_pairs) {
            const uint32_t gp = first_pair + q;
            const uint32_t r = gp / nh, h = gp % nh;
            v = __ldg(reinterpret_cast<const float4*>(p.q + ((static_cast<size_t>(seq) * p.rows + r) * p.q_heads + head0 + h) * D) + c);
        }
        *reinterpret_cast<float4*>(q_s + q * LD + (c << 2)) = v;
    }

    // This thread's two pairs: rows g and g + 8 of the warp's m16 tile.
    const int64_t rel0 = static_cast<int64_t>(blk_lo) + k0;
    int64_t vis_lo[2], vis_hi[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const uint32_t q = pb * 16 + g + 8 * e;
        const bool live = q < cta_pairs;
        const uint32_t ppos = sd.q_pos0 + (first_pair + (live ? q : 0u)) / nh;
        uint32_t abs_lo = sd.kv_lo;
        if (window != 0 && ppos + 1 > window) abs_lo = max(abs_lo, ppos + 1 - window);
        vis_lo[e] = live ? static_cast<int64_t>(abs_lo) - rel0 : 0;
        vis_hi[e] = live ? static_cast<int64_t>(ppos) + 1 - rel0 : 0;
    }

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float sl = p.scale * kLog2e;
    const float* qrow0 = q_s + (pb * 16 + g) * LD + t;
    const float* qrow1 = qrow0 + 8 * LD;

    for (uint32_t tile = 0; tile < ntiles; ++tile) {
        cp_async_wait<kStages - 2>();
        __syncthreads();  // the tile (and, the first time, the queries) landed; the stage refilled below is free
        if (tile + kStages - 1 < ntiles) load_tile(tile + kStages - 1);
        cp_async_commit();

        const uint32_t stage = tile % kStages;
        const float* kt = tiles + stage * 2 * kTileFloats;
        const float* vt = kt + kTileFloats;
        const int wrow0 = ksub * KW;  // this warp's first key row inside the tile
        const float* kfrag = kt + (wrow0 + g) * LD + t;          // K fragment base: key row g, channel slot t
        const float* vfrag = vt + (wrow0 + 2 * t) * LD + g;      // V fragment base: key row 2t, channel g

        // S(16 pairs x KW keys) = Q(16 x D) * K^T
        float s[KW / 8][4];
#pragma unroll
        for (int j = 0; j < KW / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t ah[4], al[4];
            const int c0 = 8 * ks, c1 = 8 * ks + 4;
            split_tf32(qrow0[c0], ah[0], al[0]);
            split_tf32(qrow1[c0], ah[1], al[1]);
            split_tf32(qrow0[c1], ah[2], al[2]);
            split_tf32(qrow1[c1], ah[3], al[3]);
#pragma unroll
            for (int jn = 0; jn < KW / 8; ++jn) {
                const float* krow = kfrag + 8 * jn * LD;
                uint32_t bh[2], bl[2];
                split_tf32(krow[c0], bh[0], bl[0]);
                split_tf32(krow[c1], bh[1], bl[1]);
                mma3(s[jn], ah, al, bh, bl);
            }
        }
        // scale, causal / window mask, online softmax for the thread's two pairs.  The visible columns of this
        // warp's KW keys are [c_lo, c_hi) per pair; a tile inside every pair's range needs no mask at all.
        float mx[2] = {-INFINITY, -INFINITY};
        int c_lo[2], c_hi[2];
        {
            const int64_t base = static_cast<int64_t>(tile) * kF32Tile + wrow0;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                c_lo[e] = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(KW), vis_lo[e] - base)));
                c_hi[e] = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(KW), vis_hi[e] - base)));
            }
        }
        const bool interior = __all_sync(0xffffffffu, c_lo[0] == 0 && c_lo[1] == 0 && c_hi[0] == KW && c_hi[1] == KW);
        if (interior) {
#pragma unroll
            for (int j = 0; j < KW / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    s[j][c] *= sl;
                    mx[c >> 1] = fmaxf(mx[c >> 1], s[j][c]);
                }
        } else {
#pragma unroll
            for (int j = 0; j < KW / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int e = c >> 1;
                    const int col = 8 * j + 2 * t + (c & 1);
                    const float v = (col >= c_lo[e] && col < c_hi[e]) ? s[j][c] * sl : -INFINITY;
                    s[j][c] = v;
                    mx[e] = fmaxf(mx[e], v);
                }
        }
        float m_use[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
            const float m_new = fmaxf(m[e], mx[e]);
            m_use[e] = (m_new == -INFINITY) ? 0.f : m_new;  // nothing visible yet: weights stay zero
            const float corr = fast_exp2(m[e] - m_use[e]);
            m[e] = m_new;
            l[e] *= corr;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                o[i][2 * e] *= corr;
                o[i][2 * e + 1] *= corr;
            }
        }
        // O(16 x D) += P(16 x KW keys) * V(KW keys x D), eight keys at a time.  The product's k slots t and t + 4
        // are given keys 2t and 2t + 1 of the group: exactly the two columns of S this thread already holds.
#pragma unroll
        for (int kg = 0; kg < KW / 8; ++kg) {
            const float p00 = fast_exp2(s[kg][0] - m_use[0]), p01 = fast_exp2(s[kg][1] - m_use[0]);
            const float p10 = fast_exp2(s[kg][2] - m_use[1]), p11 = fast_exp2(s[kg][3] - m_use[1]);
            l[0] += p00 + p01;
            l[1] += p10 + p11;
            uint32_t ph[4], pl[4];
            split_tf32(p00, ph[0], pl[0]);
            split_tf32(p10, ph[1], pl[1]);
            split_tf32(p01, ph[2], pl[2]);
            split_tf32(p11, ph[3], pl[3]);
            const float* vrow = vfrag + 8 * kg * LD;
#pragma unroll
            for (int jn = 0; jn < NT; ++jn) {
                uint32_t vh[2], vl[2];
                split_tf32(vrow[8 * jn], vh[0], vl[0]);
                split_tf32(vrow[LD + 8 * jn], vh[1], vl[1]);
                mma3(o[jn], ph, pl, vh, vl);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with the tiles: their place now takes the warps' results

    // Warp results into shared memory: res_o[warp][16][D] (unnormalised), res_m / res_l [warp][16].
    float* res_o = tiles;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
        float* orow = res_o + (warp * 16 + g + 8 * e) * D;
#pragma unroll
        for (int i = 0; i < NT; ++i) *reinterpret_cast<float2*>(orow + 8 * i + 2 * t) = make_float2(o[i][2 * e], o[i][2 * e + 1]);
        if (t == 0) {
            res_m[warp][g + 8 * e] = m[e];
            res_l[warp][g + 8 * e] = l[e];
        }
    }
    __syncthreads();

    // The CTA's result per pair: the WK warps that shared the pair's keys, merged.
    const uint32_t HYP = p.layer.kv_heads * p.gchunks * pchunks;
    const size_t cell = static_cast<size_t>(seq) * HYP + hy * pchunks + pc;
    const size_t slot = cell * p.splits + split;
    for (uint32_t idx = tid; idx < cta_pairs * D; idx += kF32Threads) {
        const uint32_t q = idx / D, dd = idx % D;
        const uint32_t w0 = (q / 16) * WK, r = q % 16;
        float M = -INFINITY;
#pragma unroll
        for (int j = 0; j < WK; ++j) M = fmaxf(M, res_m[w0 + j][r]);
        float O = 0.f, L = 0.f;
#pragma unroll
        for (int j = 0; j < WK; ++j) {
            const float mj = res_m[w0 + j][r];
            const float w = (mj == -INFINITY) ? 0.f : fast_exp2(mj - M);
            O += w * res_o[((w0 + j) * 16 + r) * D + dd];
            L += w * res_l[w0 + j][r];
        }
        if (parts == 1) {
            const uint32_t gp = first_pair + q;
            p.out[((static_cast<size_t>(seq) * p.rows + gp / nh) * p.q_heads + head0 + gp % nh) * D + dd] = O / L;
        } else {
            p.part_o[(slot * PC + q) * D + dd] = O;
            if (dd == 0) {
                p.part_ml[(slot * PC + q) * 2] = M;
                p.part_ml[(slot * PC + q) * 2 + 1] = L;
            }
        }
    }
    if (parts == 1) return;
    __syncthreads();
    if (tid == 0) {
        __threadfence();  // cumulative over the CTA's stores above (ordered before the barrier)
        const unsigned int ticket = atomicAdd(p.tickets + cell, 1u);
        s_flag = (ticket == parts - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_flag == 0) return;
    __threadfence();
    // The last arrival merges every part of the block (log-sum-exp).  First every part's (max, sum) pairs into shared
    // memory in one round trip, from them the parts' weights per pair, w[part][pair] = 2^(max_part - max_all) / sum;
    // then every output channel as a weighted sum over the parts, the loads of up to four parts in flight together.
    const float* all_o = p.part_o + cell * p.splits * PC * D;
    const float2* all_ml = reinterpret_cast<const float2*>(p.part_ml) + cell * p.splits * PC;
    // (both arrays start where the queries were: at most kF32MaxParts x PC x 12 bytes, inside the CTA's allocation)
    float* w_s = q_s;                                             // [parts][PC] weights
    float2* ml_s = reinterpret_cast<float2*>(q_s + parts * PC);   // [parts][PC] (max, sum) pairs
    static_assert(static_cast<size_t>(kF32MaxParts) * PC * 12 <= (static_cast<size_t>(PC) + kStages * 2 * kF32Tile) * LD * 4,
                  "merge scratch exceeds the CTA's shared memory");
    for (uint32_t i = tid; i < parts * PC; i += kF32Threads) ml_s[i] = __ldcg(all_ml + i);  // one round trip for all
    __syncthreads();
    if (tid < cta_pairs) {
        float M = -INFINITY;
        for (uint32_t sp = 0; sp < parts; ++sp) M = fmaxf(M, ml_s[sp * PC + tid].x);
        float L = 0.f;
        for (uint32_t sp = 0; sp < parts; ++sp) {
            const float2 ml = ml_s[sp * PC + tid];
            const float w = (ml.x == -INFINITY) ? 0.f : fast_exp2(ml.x - M);
            w_s[sp * PC + tid] = w;
            L += w * ml.y;
        }
        const float inv = 1.f / L;
        for (uint32_t sp = 0; sp < parts; ++sp) w_s[sp * PC + tid] *= inv;
    }
    __syncthreads();
    constexpr int kOutPerThread = PC * D / kF32Threads;
    constexpr int kPartBatch = kOutPerThread <= 8 ? 4 : (kOutPerThread <= 16 ? 2 : 1);  // parts whose loads fly together
    float acc[kOutPerThread];
#pragma unroll
    for (int i = 0; i < kOutPerThread; ++i) acc[i] = 0.f;
    for (uint32_t sp0 = 0; sp0 < parts; sp0 += kPartBatch) {
        float v[kPartBatch][kOutPerThread];
#pragma unroll
        for (int b = 0; b < kPartBatch; ++b) {
            const uint32_t sp = min(sp0 + b, parts - 1);  // a repeated part past the end gets weight zero below
            const float* src = all_o + static_cast<size_t>(sp) * PC * D;
#pragma unroll
            for (int i = 0; i < kOutPerThread; ++i) {
                const uint32_t idx = tid + i * kF32Threads;
                v[b][i] = idx < cta_pairs * D ? __ldcg(src + idx) : 0.f;
            }
        }
#pragma unroll
        for (int b = 0; b < kPartBatch; ++b) {
            const bool real = sp0 + b < parts;
#pragma unroll
            for (int i = 0; i < kOutPerThread; ++i) {
                const uint32_t idx = tid + i * kF32Threads;
                const float w = (real && idx < cta_pairs * D) ? w_s[(sp0 + b) * PC + idx / D] : 0.f;
                acc[i] += w * v[b][i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kOutPerThread; ++i) {
        const uint32_t idx = tid + i * kF32Threads;
        if (idx < cta_pairs * D) {
            const uint32_t gp = first_pair + idx / D;
            p.out[((static_cast<size_t>(seq) * p.rows + gp / nh) * p.q_heads + head0 + gp % nh) * D + idx % D] = acc[i];
        }
    }
    if (tid == 0) p.tickets[cell] = 0u;
}

// grid = (key parts, head chunks x pair blocks, sequences)
template <int D, int WK>
__global__ void __launch_bounds__(kF32Threads, D == 64 ? 4 : 2) attn_f32_kernel(const __grid_constant__ AttnLaunch p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr uint32_t PC = 16 * (4 / WK);
    const uint32_t gheads = min(p.group, static_cast<uint32_t>(kHeadsPerCta));
    const uint32_t pchunks = (p.rows * gheads + PC - 1) / PC;
    // the pair blocks of a head chunk are handed out last block first: under the causal bound it has the longest
    // key range, and the CTAs placed last should be the short ones
    f32_block<D, WK>(p, smem, blockIdx.z, blockIdx.y / pchunks, pchunks - 1 - blockIdx.y % pchunks, pchunks, blockIdx.x);
}

template <int D, int WK>
constexpr size_t f32_smem_bytes() {
    return (static_cast<size_t>(16 * (4 / WK)) * (D + 4) + static_cast<size_t>(kF32Stages) * 2 * kF32Tile * (D + 4)) * sizeof(float);
}

template <int D, int WK>
cudaError_t configure_one() {
    return cudaFuncSetAttribute(attn_f32_kernel<D, WK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(f32_smem_bytes<D, WK>()));
}

template <int D, int WK>
void launch_one(const AttnLaunch& p, dim3 grid, cudaStream_t s) {
    attn_f32_kernel<D, WK><<<grid, kF32Threads, f32_smem_bytes<D, WK>(), s>>>(p);
}

}  // namespace

bool attn_f32_supported(uint32_t head_dim, uint32_t rows) { return rows >= 1 && (head_dim == 64 || head_dim == 128); }

// (row, head) pairs one CTA owns: 16 when the whole group's block fits (the four warps then share its keys), else 64.
uint32_t attn_f32_pairs_per_cta(uint32_t rows, uint32_t group) {
    const uint32_t nh = group < static_cast<uint32_t>(kHeadsPerCta) ? group : kHeadsPerCta;
    return static_cast<uint64_t>(rows) * nh <= 16 ? 16u : 64u;
}

uint32_t attn_f32_pair_chunks(uint32_t rows, uint32_t group) {
    const uint32_t nh = group < static_cast<uint32_t>(kHeadsPerCta) ? group : kHeadsPerCta;
    const uint32_t pcta = attn_f32_pairs_per_cta(rows, group);
    return static_cast<uint32_t>((static_cast<uint64_t>(rows) * nh + pcta - 1) / pcta);
}

uint32_t attn_f32_max_parts() { return kF32MaxParts; }

cudaError_t configure_attn_f32() {
    cudaError_t e = configure_one<64, 1>();
    if (e == cudaSuccess) e = configure_one<64, 4>();
    if (e == cudaSuccess) e = configure_one<128, 1>();
    if (e == cudaSuccess) e = configure_one<128, 4>();
    return e;
}

cudaError_t launch_attn_f32(const AttnLaunch& p, cudaStream_t s, uint64_t* launches) {
    if (!attn_f32_supported(p.layer.head_dim, p.rows) || p.splits == 0 || p.splits > kF32MaxParts) return cudaErrorInvalidValue;
    const uint32_t pchunks = attn_f32_pair_chunks(p.rows, p.group);
    const bool shared_keys = attn_f32_pairs_per_cta(p.rows, p.group) == 16;
    const dim3 grid(p.splits, p.layer.kv_heads * p.gchunks * pchunks, p.n_seqs);
    if (grid.y > 65535u) return cudaErrorInvalidValue;
    if (p.layer.head_dim == 64) {
        if (shared_keys) launch_one<64, 4>(p, grid, s); else launch_one<64, 1>(p, grid, s);
    } else {
        if (shared_keys) launch_one<128, 4>(p, grid, s); else launch_one<128, 1>(p, grid, s);
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk
