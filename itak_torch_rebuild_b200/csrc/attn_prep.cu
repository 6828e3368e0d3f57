// Attention preparation on the device: the per-head RMSNorm of the Q and K rows and their rotary rotation, in
// one launch over every head row of the call, ahead of the append + attention kernels.
//
// Stands in for the reference's fused preparation K9 (crates/wgpu-compute/src/kernels/k9_attn_prep.rs:74-236:
// weighted RMSNorm per head row at the file eps, adjacent-pair rotation at position * base^(-2i/rotary_dim),
// rows then appended) and for the rotation the CPU backend applies inside its attention step
// (crates/cpu-compute/src/cpu.rs:598-622).  The rows' append stays with the attention kernels, which store the
// prepared K rows and the V rows themselves.
//
// Arithmetic follows the CPU reference rather than the f32 shader: the mean of squares and the normalised value
// in f64, rounded once to f32 (crates/torch-math/src/norm.rs:21-53); the angle, its sine and cosine and the
// rotated pair in f64, rounded once to f32 (crates/torch-math/src/rope_interleaved.rs:65-117, rope.rs:63-117).
// The inverse frequencies base^(-2i/rotary_dim) come from the host as f64 (one table per layer), so the only
// differences from the CPU path are the order of the f64 sum of squares and the last bit of sin / cos.
//
// One warp owns one head row (head_dim <= 256): it sums the squares with shuffles, writes the normalised row to
// its slice of shared memory, and every lane rotates the pairs it owns from there.  Bound: launch latency - a
// decode step touches n_seqs x (q_heads + kv_heads) x head_dim x 8 bytes.
#include <cstdio>

#include "kernels.cuh"

namespace itk {

namespace {

constexpr int kPrepWarps = 4;
constexpr int kPrepMaxD = 256;

__global__ void __launch_bounds__(kPrepWarps * 32) prep_rows_kernel(const __grid_constant__ PrepLaunch p) {
    __shared__ float rows_s[kPrepWarps][kPrepMaxD];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t heads = p.q_heads + p.kv_heads;
    const uint64_t total = static_cast<uint64_t>(p.n_seqs) * p.rows * heads;
    const uint64_t unit = static_cast<uint64_t>(blockIdx.x) * kPrepWarps + warp;
    if (unit >= total) return;  // whole warps leave; no CTA barrier follows
    const uint32_t head = static_cast<uint32_t>(unit % heads);
    const uint64_t srow = unit / heads;  // sequence * rows + row
    const uint32_t seq = static_cast<uint32_t>(srow / p.rows), row = static_cast<uint32_t>(srow % p.rows);
    const bool is_q = head < p.q_heads;
    const uint32_t D = p.head_dim;
    const size_t off = is_q ? (srow * p.q_heads + head) * D : (srow * p.kv_heads + (head - p.q_heads)) * D;
    const float* src = (is_q ? p.q_in : p.k_in) + off;
    float* dst = (is_q ? p.q_out : p.k_out) + off;
    const float* w = is_q ? p.q_w : p.k_w;
    float* mine = rows_s[warp];

    // RMSNorm of the head row (skipped without a weight vector).
    float x[kPrepMaxD / 32];
    double sq = 0.0;
#pragma unroll
    for (int j = 0; j < kPrepMaxD / 32; ++j) {
        const uint32_t d = lane + 32 * j;
        x[j] = d < D ? src[d] : 0.f;
        sq += static_cast<double>(x[j]) * static_cast<double>(x[j]);
    }
    if (w != nullptr) {
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, s);
        const double inv_rms = 1.0 / sqrt(sq / static_cast<double>(D) + static_cast<double>(p.eps));
#pragma unroll
        for (int j = 0; j < kPrepMaxD / 32; ++j) {
            const uint32_t d = lane + 32 * j;
            if (d < D) x[j] = static_cast<float>(static_cast<double>(x[j]) * inv_rms * static_cast<double>(w[d]));
        }
    }
    const uint32_t rot = p.rotary_dim;
    if (rot == 0) {
#pragma unroll
        for (int j = 0; j < kPrepMaxD / 32; ++j) {
            const uint32_t d = lane + 32 * j;
            if (d < D) dst[d] = x[j];
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < kPrepMaxD / 32; ++j) {
        const uint32_t d = lane + 32 * j;
        if (d < D) mine[d] = x[j];
    }
    __syncwarp();
    // Rotation: pair i joins channels (2i, 2i + 1) or (i, i + rot / 2); channels past rotary_dim pass through.
    const double pos = static_cast<double>(p.pos0[seq] + row);
    const uint32_t half = rot / 2;
    for (uint32_t i = lane; i < half; i += 32) {
        const uint32_t a = p.pairing == 0 ? 2 * i : i, b = p.pairing == 0 ? 2 * i + 1 : i + half;
        double s, c;
        sincos(pos * p.inv_freq[i], &s, &c);
        const double u = mine[a], v = mine[b];
        dst[a] = static_cast<float>(u * c - v * s);
        dst[b] = static_cast<float>(u * s + v * c);
    }
    for (uint32_t d = rot + lane; d < D; d += 32) dst[d] = mine[d];
}

// In-place rotation of `rows` x `heads` head rows at per-row positions read from a device array: the rotate half of
// the reference's K17 (crates/wgpu-compute/src/kernels/k17_dflash.rs:78-107), whose two call sites see different
// position sources (an inject chunk's caller-supplied positions, a block's start..start+rows span).  One thread per
// pair; a pair's two channels are read and written by that thread alone, so the rotation is safe in place.  Angle,
// sine, cosine and the products in f64, rounded once (crates/torch-math/src/rope.rs:63-117).
__global__ void rope_rows_kernel(float* x, const uint32_t* positions, uint32_t rows, uint32_t heads, uint32_t head_dim,
                                 uint32_t rotary_dim, uint32_t pairing, double base) {
    const uint32_t half = rotary_dim / 2;
    const uint64_t per_row = static_cast<uint64_t>(heads) * half;
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<uint64_t>(rows) * per_row) return;
    const uint32_t row = static_cast<uint32_t>(idx / per_row);
    const uint32_t rem = static_cast<uint32_t>(idx % per_row);
    const uint32_t head = rem / half, i = rem % half;
    const double angle = static_cast<double>(positions[row]) *
                         pow(base, -static_cast<double>(2 * i) / static_cast<double>(rotary_dim));
    double s, c;
    sincos(angle, &s, &c);
    float* h = x + (static_cast<size_t>(row) * heads + head) * head_dim;
    const uint32_t a = pairing == 0 ? 2 * i : i, b = pairing == 0 ? 2 * i + 1 : i + half;
    const double u = h[a], v = h[b];
    h[a] = static_cast<float>(u * c - v * s);
    h[b] = static_cast<float>(u * s + v * c);
}

}  // namespace

cudaError_t launch_prep(const PrepLaunch& p, cudaStream_t s, uint64_t* launches) {
    if (p.n_seqs == 0 || p.n_seqs > static_cast<uint32_t>(kMaxSeqsPerLaunch) || p.rows == 0 || p.head_dim == 0 ||
        p.head_dim > static_cast<uint32_t>(kPrepMaxD) || p.rotary_dim > p.head_dim || (p.rotary_dim & 1u) != 0 ||
        (p.rotary_dim != 0 && p.inv_freq == nullptr))
        return cudaErrorInvalidValue;
    const uint64_t total = static_cast<uint64_t>(p.n_seqs) * p.rows * (p.q_heads + p.kv_heads);
    const uint64_t blocks = (total + kPrepWarps - 1) / kPrepWarps;
    if (blocks == 0 || blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    prep_rows_kernel<<<static_cast<unsigned int>(blocks), kPrepWarps * 32, 0, s>>>(p);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk

// Refusals follow check_rotate (crates/wgpu-compute/src/kernels/k17_dflash.rs:255-271) and the CPU function's own
// (crates/torch-math/src/rope.rs:70-95), by the same names.
extern "C" int itk_rope_rows(float* d_x, const uint32_t* d_positions, uint32_t rows, uint32_t heads, uint32_t head_dim,
                             uint32_t rotary_dim, uint32_t pairing, float base, void* cuda_stream, char* error_text,
                             size_t error_text_len) {
    auto refuse = [&](const char* fmt, unsigned long long a = 0, unsigned long long b = 0) {
        if (error_text && error_text_len) snprintf(error_text, error_text_len, fmt, a, b);
        return 101;  // ITK_ERR_INVALID_ARGUMENT
    };
    if (error_text && error_text_len) error_text[0] = '\0';
    if (rows == 0 || heads == 0) return refuse("rotate needs at least one row and head, got rows %llu, heads %llu", rows, heads);
    if (head_dim < 2 || head_dim % 2 != 0) return refuse("head_dim %llu must be even and at least 2", head_dim);
    if (rotary_dim < 2 || rotary_dim % 2 != 0 || rotary_dim > head_dim)
        return refuse("rope: rotary_dim must be even, >= 2, and <= head_dim");
    if (!(base > 1.0f) || base > 3.0e38f) return refuse("rope: base must be finite and > 1");
    if (pairing > 1) return refuse("rope: pairing is 0 (adjacent) or 1 (half split)");
    if (!d_x || !d_positions) return refuse("null pointer argument");
    const unsigned long long pairs = static_cast<unsigned long long>(rows) * heads * (rotary_dim / 2);
    const unsigned long long blocks = (pairs + 127) / 128;
    if (blocks > 0x7fffffffull) return refuse("rows x heads x rotary_dim = %llu pairs is too large", pairs);
    itk::rope_rows_kernel<<<static_cast<unsigned int>(blocks), 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        d_x, d_positions, rows, heads, head_dim, rotary_dim, pairing, static_cast<double>(base));
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        if (error_text && error_text_len) snprintf(error_text, error_text_len, "rotate launch failed: %s", cudaGetErrorString(e));
        return 100;  // ITK_ERR_CUDA
    }
    return 0;
}
