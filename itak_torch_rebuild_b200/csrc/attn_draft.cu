// Draft-model (DFlash) attention: the visible set is a position-addressed, possibly sparse set of committed rows
// plus the current block's own K/V rows, non-causal unless asked, under a sliding-window mask over absolute
// positions.
//
// Stands in for the attention half of the reference's K17
// (crates/wgpu-compute/src/kernels/k17_dflash.rs:109-251) and follows the CPU draft model it mirrors
// (crates/dflash/src/model.rs:388-466): for query row r at position p = block_start + r, key kp is visible unless
// (causal and kp > p) or (sliding and kp <= p - window, in signed arithmetic); committed rows come first, in the
// order of the position list, then the block rows in order; score = (q . k) * scale, softmax over the visible
// set, output = sum of weight * v.  f32 throughout.
//
// The committed arrays are POSITION-ADDRESSED like the reference's device buffers: the row of position kp starts
// at kp * kv_heads * key_len (values: kp * kv_heads * value_len); `positions` lists which rows exist.
//
// One CTA serves one (query row, query head): its four warps take every fourth key of the set, lanes share the
// dot product and own value channels lane, lane + 32, ...; each warp keeps an online-softmax state, merged through
// shared memory at the end.  A draft block is a handful of rows against a few thousand committed positions, all of
// it L2-resident, so the kernel is latency-bound by design; what matters is that it never leaves the device.
#include <cstdio>

#include "attn_common.cuh"

namespace itk {

namespace {

constexpr int kDraftWarps = 4;
constexpr int kDraftMaxLen = 256;  // key_len and value_len bound (8 channels per lane)
constexpr int kDraftPerLane = kDraftMaxLen / 32;

struct DraftLaunch {
    const float* q;           // [rows][q_heads][key_len]
    const float* ck;          // committed keys, position-addressed
    const float* cv;          // committed values, position-addressed
    const uint32_t* cpos;     // [committed] positions held
    const float* bk;          // [block_rows][kv_heads][key_len]
    const float* bv;          // [block_rows][kv_heads][value_len]
    float* out;               // [rows][q_heads][value_len]
    uint32_t rows, q_heads, kv_heads, group, key_len, value_len, block_rows, block_start, committed;
    uint32_t causal, sliding, window;
    float scale;
};

__device__ __forceinline__ bool draft_visible(const DraftLaunch& p, uint32_t kp, uint32_t qp) {
    if (p.causal != 0 && kp > qp) return false;
    if (p.sliding != 0 && static_cast<int32_t>(kp) <= static_cast<int32_t>(qp) - static_cast<int32_t>(p.window))
        return false;
    return true;
}

__global__ void __launch_bounds__(kDraftWarps * 32) draft_attention_kernel(const __grid_constant__ DraftLaunch p) {
    __shared__ float s_q[kDraftMaxLen];
    __shared__ float s_m[kDraftWarps], s_l[kDraftWarps];
    __shared__ float s_o[kDraftWarps][kDraftMaxLen];
    const uint32_t row = blockIdx.x / p.q_heads, qh = blockIdx.x % p.q_heads;
    const uint32_t kvh = qh / p.group;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t qp = p.block_start + row;
    const size_t k_width = static_cast<size_t>(p.kv_heads) * p.key_len, v_width = static_cast<size_t>(p.kv_heads) * p.value_len;
    for (uint32_t d = threadIdx.x; d < p.key_len; d += blockDim.x)
        s_q[d] = p.q[(static_cast<size_t>(row) * p.q_heads + qh) * p.key_len + d];
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[kDraftPerLane];
#pragma unroll
    for (int j = 0; j < kDraftPerLane; ++j) acc[j] = 0.f;
    const uint32_t total = p.committed + p.block_rows;
    for (uint32_t idx = warp; idx < total; idx += kDraftWarps) {
        uint32_t kp;
        const float *krow, *vrow;
        if (idx < p.committed) {
            kp = p.cpos[idx];
            krow = p.ck + kp * k_width + kvh * p.key_len;
            vrow = p.cv + kp * v_width + kvh * p.value_len;
        } else {
            const uint32_t brow = idx - p.committed;
            kp = p.block_start + brow;
            krow = p.bk + brow * k_width + kvh * p.key_len;
            vrow = p.bv + brow * v_width + kvh * p.value_len;
        }
        if (!draft_visible(p, kp, qp)) continue;  // warp-uniform
        float part = 0.f;
        for (uint32_t d = lane; d < p.key_len; d += 32) part += s_q[d] * krow[d];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
        const float score = part * p.scale;
        const float m_new = fmaxf(m, score);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first visible key
        const float w = expf(score - m_new);
        m = m_new;
        l = l * corr + w;
#pragma unroll
        for (int j = 0; j < kDraftPerLane; ++j) {
            const uint32_t d = lane + 32 * j;
            if (d < p.value_len) acc[j] = acc[j] * corr + w * vrow[d];
        }
    }
    if (lane == 0) {
        s_m[warp] = m;
        s_l[warp] = l;
    }
#pragma unroll
    for (int j = 0; j < kDraftPerLane; ++j) {
        const uint32_t d = lane + 32 * j;
        if (d < p.value_len) s_o[warp][d] = acc[j];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDraftWarps; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f, a[kDraftWarps];
#pragma unroll
    for (int w = 0; w < kDraftWarps; ++w) {
        a[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);
        L += a[w] * s_l[w];
    }
    // The query's own block row is always visible, so L > 0; an empty set would give zeros, as in the reference.
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (uint32_t d = threadIdx.x; d < p.value_len; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kDraftWarps; ++w) o += a[w] * s_o[w][d];
        p.out[(static_cast<size_t>(row) * p.q_heads + qh) * p.value_len + d] = o * inv;
    }
}

int draft_refuse(char* text, size_t text_len, const char* fmt, unsigned long long a = 0, unsigned long long b = 0) {
    if (text && text_len) snprintf(text, text_len, fmt, a, b);
    return 101;  // ITK_ERR_INVALID_ARGUMENT
}

}  // namespace

}  // namespace itk

// Geometry refusals follow check_attend (crates/wgpu-compute/src/kernels/k17_dflash.rs:276-316), by the same names.
extern "C" int itk_draft_attention(const float* d_q, const float* d_committed_k, const float* d_committed_v,
                                   const uint32_t* d_committed_positions, uint32_t committed, const float* d_block_k,
                                   const float* d_block_v, uint32_t block_start, uint32_t rows, uint32_t block_rows,
                                   uint32_t q_heads, uint32_t kv_heads, uint32_t key_len, uint32_t value_len,
                                   uint32_t causal, uint32_t sliding, uint32_t window, float scale, float* d_out,
                                   void* cuda_stream, char* error_text, size_t error_text_len) {
    using namespace itk;
    if (error_text && error_text_len) error_text[0] = '\0';
    if (rows == 0 || block_rows == 0)
        return draft_refuse(error_text, error_text_len,
                            "draft attention needs at least one query row and one block row, got rows %llu, block_rows %llu",
                            rows, block_rows);
    if (q_heads == 0 || kv_heads == 0 || q_heads % kv_heads != 0)
        return draft_refuse(error_text, error_text_len,
                            "q_heads %llu must be a whole multiple of kv_heads %llu, both non-zero", q_heads, kv_heads);
    if (key_len == 0) return draft_refuse(error_text, error_text_len, "key_len is zero");
    if (key_len > static_cast<uint32_t>(kDraftMaxLen))
        return draft_refuse(error_text, error_text_len, "key_len %llu outside the kernel's supported range 1..=%llu",
                            key_len, static_cast<unsigned long long>(kDraftMaxLen));
    if (value_len == 0 || value_len > static_cast<uint32_t>(kDraftMaxLen))
        return draft_refuse(error_text, error_text_len, "value_len %llu outside the kernel's supported range 1..=%llu",
                            value_len, static_cast<unsigned long long>(kDraftMaxLen));
    if (!d_q || !d_block_k || !d_block_v || !d_out || (committed != 0 && (!d_committed_k || !d_committed_v || !d_committed_positions)))
        return draft_refuse(error_text, error_text_len, "null pointer argument");
    const unsigned long long blocks = static_cast<unsigned long long>(rows) * q_heads;
    if (blocks > 0x7fffffffull) return draft_refuse(error_text, error_text_len, "rows x q_heads = %llu is too large", blocks);
    DraftLaunch p{};
    p.q = d_q;
    p.ck = d_committed_k;
    p.cv = d_committed_v;
    p.cpos = d_committed_positions;
    p.bk = d_block_k;
    p.bv = d_block_v;
    p.out = d_out;
    p.rows = rows;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.group = q_heads / kv_heads;
    p.key_len = key_len;
    p.value_len = value_len;
    p.block_rows = block_rows;
    p.block_start = block_start;
    p.committed = committed;
    p.causal = causal;
    p.sliding = sliding;
    p.window = window;
    p.scale = scale;
    draft_attention_kernel<<<static_cast<unsigned int>(blocks), kDraftWarps * 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(p);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        if (error_text && error_text_len)
            snprintf(error_text, error_text_len, "draft attention launch failed: %s", cudaGetErrorString(e));
        return 100;  // ITK_ERR_CUDA
    }
    return 0;
}
