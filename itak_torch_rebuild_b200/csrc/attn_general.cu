// General GQA attention over the resident cache: any head_dim up to 256, any
// number of query rows, f32 or f16 cache elements, global or sliding layers.
//
// This is the path for the reference's own CPU-sized configurations (f32 cache,
// crates/attention/src/cache.rs:11-15) and for every shape the tensor-core
// kernels do not take.  It follows gqa_attention
// (crates/attention/src/attention.rs:104-215) closely: per query row the
// visible keys are positions (p - window, p] intersected with what is stored,
// each score is a dot product accumulated in ascending channel order in f32
// and multiplied by the scale, the softmax is max-subtracted, and the output is
// the weighted sum of value rows.  The only departures are the online
// (tile-by-tile) form of the softmax and exp2 with a log2(e)-prescaled score.
//
// One CTA per (query row, KV head chunk of <= 8 query heads, split of the key
// range).  Per 128-key tile: thread i owns key i for the scores (all heads of
// the group reuse the key row it reads), then thread j owns output channel(s)
// (head, d) for the value accumulation, reading value rows coalesced.
// Bound: HBM for long contexts; at the f32 configuration (2 FMA per byte) the
// fp32 pipe has ~3x headroom.
#include "attn_common.cuh"

namespace itk {

namespace {

constexpr int kGenThreads = 128;
constexpr int kGenTile = 128;       // keys per tile = one per thread
constexpr int kGenMaxD = 256;
constexpr int kGenOutPerThread = kHeadsPerCta * kGenMaxD / kGenThreads;  // 16

__device__ __forceinline__ float kv_load(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float kv_load(const __half* p, size_t i) { return __half2float(p[i]); }

template <typename KV>
__global__ void __launch_bounds__(kGenThreads) attn_general_kernel(const __grid_constant__ AttnLaunch p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t D = p.layer.head_dim;
    float* q_s = reinterpret_cast<float*>(smem);          // [8][D]
    float* sc = q_s + kHeadsPerCta * D;                   // [8][128] scores, then weights
    float* fo = sc + kHeadsPerCta * kGenTile;             // [8][D]
    float* m_s = fo + kHeadsPerCta * D;                   // [8]
    float* l_s = m_s + kHeadsPerCta;                      // [8]
    float* corr = l_s + kHeadsPerCta;                     // [8]
    int* flag = reinterpret_cast<int*>(corr + kHeadsPerCta);
    float* wscratch = corr + kHeadsPerCta + 4;            // merge weights: [2][256][8] + [8]

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t split = blockIdx.x, hy = blockIdx.y, unit = blockIdx.z;
    const uint32_t seq = unit / p.rows, r = unit % p.rows;
    const SeqDesc sd = p.seq[seq];
    const uint32_t kvh = hy / p.gchunks, gc = hy % p.gchunks;
    const uint32_t head0 = kvh * p.group + gc * kHeadsPerCta;
    const uint32_t nh = min(static_cast<uint32_t>(kHeadsPerCta), p.group - gc * kHeadsPerCta);
    const uint32_t ring = p.layer.ring;

    // Visible positions of this row: [lo, hi).
    const uint32_t pr = sd.q_pos0 + r;
    const uint32_t hi = pr + 1;
    uint32_t lo = sd.kv_lo;
    if (p.layer.window != 0 && hi > p.layer.window) lo = max(lo, hi - p.layer.window);
    const uint32_t n = hi - lo;
    uint32_t chunk = (n + p.splits - 1) / p.splits;
    chunk = (chunk + kGenTile - 1) / kGenTile * kGenTile;
    const uint32_t k0 = min(n, split * chunk);
    const uint32_t k1 = min(n, k0 + chunk);
    const uint32_t span = k1 - k0;
    const uint32_t s0 = (lo + k0) % ring;

    const size_t stream = (static_cast<size_t>(sd.slot) * p.layer.kv_heads + kvh) * ring * D;
    const KV* kbase = static_cast<const KV*>(p.layer.k) + stream;
    const KV* vbase = static_cast<const KV*>(p.layer.v) + stream;

    const float* qrow = p.q + (static_cast<size_t>(unit) * p.q_heads + head0) * D;
    for (uint32_t i = tid; i < nh * D; i += kGenThreads) q_s[i] = qrow[i];
    if (tid < kHeadsPerCta) {
        m_s[tid] = -INFINITY;
        l_s[tid] = 0.f;
    }
    float o[kGenOutPerThread];
#pragma unroll
    for (int i = 0; i < kGenOutPerThread; ++i) o[i] = 0.f;
    const float sl = p.scale * kLog2e;
    __syncthreads();

    for (uint32_t t0 = 0; t0 < span; t0 += kGenTile) {
        const uint32_t tile_n = min(static_cast<uint32_t>(kGenTile), span - t0);
        // scores: thread tid owns key t0 + tid
        {
            float acc[kHeadsPerCta];
#pragma unroll
            for (int h = 0; h < kHeadsPerCta; ++h) acc[h] = 0.f;
            if (tid < tile_n) {
                uint32_t srow = s0 + t0 + tid;
                if (srow >= ring) srow -= ring;
                const KV* krow = kbase + static_cast<size_t>(srow) * D;
                for (uint32_t d = 0; d < D; ++d) {
                    const float kd = kv_load(krow, d);
#pragma unroll
                    for (int h = 0; h < kHeadsPerCta; ++h)
                        if (static_cast<uint32_t>(h) < nh) acc[h] += q_s[h * D + d] * kd;
                }
            }
#pragma unroll
            for (int h = 0; h < kHeadsPerCta; ++h) sc[h * kGenTile + tid] = tid < tile_n ? acc[h] * sl : -INFINITY;
        }
        __syncthreads();
        // per-head tile max and weights: warp w takes heads w and w + 4
        for (uint32_t h = warp; h < nh; h += kGenThreads / 32) {
            float* row = sc + h * kGenTile;
            float mx = -INFINITY;
            for (uint32_t j = lane; j < kGenTile; j += 32) mx = fmaxf(mx, row[j]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, mx);  // finite: the tile holds at least one key
            float sum = 0.f;
            for (uint32_t j = lane; j < kGenTile; j += 32) {
                const float w = fast_exp2(row[j] - m_new);
                row[j] = w;
                sum += w;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (lane == 0) {
                const float c = fast_exp2(m_old - m_new);
                corr[h] = c;
                l_s[h] = l_s[h] * c + sum;
                m_s[h] = m_new;
            }
        }
        __syncthreads();
        // outputs: thread owns channels idx = tid + 128 * i of the [nh][D] block
#pragma unroll
        for (int i = 0; i < kGenOutPerThread; ++i) {
            const uint32_t idx = tid + kGenThreads * i;
            if (idx < nh * D) {
                const uint32_t h = idx / D, d = idx % D;
                float a = o[i] * corr[h];
                const float* w = sc + h * kGenTile;
                uint32_t srow = s0 + t0;
                if (srow >= ring) srow -= ring;
                for (uint32_t j = 0; j < tile_n; ++j) {
                    a += w[j] * kv_load(vbase, static_cast<size_t>(srow) * D + d);
                    if (++srow == ring) srow = 0;
                }
                o[i] = a;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < kGenOutPerThread; ++i) {
        const uint32_t idx = tid + kGenThreads * i;
        if (idx < nh * D) fo[idx] = o[i];
    }
    __syncthreads();
    finish_unit<kGenThreads, kMaxSplits>(p, unit, hy, p.splits, split, head0, nh, D, fo, m_s, l_s, flag, wscratch);
}

size_t general_smem_bytes(uint32_t D) {
    return (static_cast<size_t>(kHeadsPerCta) * D * 2 + kHeadsPerCta * kGenTile + 3 * kHeadsPerCta + 4 +
            2 * kMaxSplits * kHeadsPerCta + kHeadsPerCta) * sizeof(float);
}

}  // namespace

cudaError_t launch_attn_general(const AttnLaunch& p, bool f16, cudaStream_t s, uint64_t* launches) {
    if (p.layer.head_dim == 0 || p.layer.head_dim > kGenMaxD) return cudaErrorInvalidValue;
    if (p.splits == 0 || p.splits > static_cast<uint32_t>(kMaxSplits)) return cudaErrorInvalidValue;
    const dim3 grid(p.splits, p.layer.kv_heads * p.gchunks, p.n_seqs * p.rows);
    const size_t smem = general_smem_bytes(p.layer.head_dim);
    if (f16)
        attn_general_kernel<__half><<<grid, kGenThreads, smem, s>>>(p);
    else
        attn_general_kernel<float><<<grid, kGenThreads, smem, s>>>(p);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk
