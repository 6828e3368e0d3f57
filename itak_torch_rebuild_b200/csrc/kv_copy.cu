// The copy paths of the resident cache: append (with the f32 -> f16 cast),
// prefix-snapshot gather and restore scatter.  All are transposes between the
// callers' position-major rows `[position][kv_head][D]` and the head-major
// device layout `[slot][kv_head][row][D]`, moved as 16-byte vectors, and all
// are bit-exact by contract.  Bound: HBM (read + write of the moved bytes);
// an append of a few rows is launch latency.
#include "kernels.cuh"
#include "kv_convert.cuh"

namespace itk {

namespace {

// Stores VEC consecutive elements starting at element offset `off`.
template <bool F16, int VEC>
__device__ __forceinline__ void store_converted(void* dst, size_t off, const float* src) {
    if constexpr (VEC == 8) {
        const float4 a = *reinterpret_cast<const float4*>(src);
        const float4 b = *reinterpret_cast<const float4*>(src + 4);
        if constexpr (F16) {
            *reinterpret_cast<uint4*>(static_cast<unsigned short*>(dst) + off) = pack8(a, b);
        } else {
            float* d = static_cast<float*>(dst) + off;
            *reinterpret_cast<float4*>(d) = a;
            *reinterpret_cast<float4*>(d + 4) = b;
        }
    } else {
        if constexpr (F16)
            static_cast<unsigned short*>(dst)[off] = f32_to_f16_bits(*src);
        else
            static_cast<float*>(dst)[off] = *src;
    }
}

// Append: rows q_pos0.. of every listed sequence, K and V, into storage rows
// position % ring.  Follows KvCache::append / LayerCache::write
// (crates/attention/src/cache.rs:181-203, 423-474) and the K5 append shader's
// slot law (crates/wgpu-compute/src/kernels/k5_rope_kv.rs:90-123).
template <bool F16, int VEC>
__global__ void __launch_bounds__(256) append_kernel(const __grid_constant__ AppendLaunch p) {
    const uint32_t dv = p.head_dim / VEC;
    const size_t per_seq = static_cast<size_t>(p.rows) * p.kv_heads * dv;
    const size_t total = per_seq * p.n_seqs;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t seq = static_cast<uint32_t>(idx / per_seq);
        size_t w = idx % per_seq;
        const uint32_t v = static_cast<uint32_t>(w % dv);
        w /= dv;
        const uint32_t h = static_cast<uint32_t>(w % p.kv_heads);
        const uint32_t r = static_cast<uint32_t>(w / p.kv_heads);
        const SeqDesc sd = p.seq[seq];
        const uint32_t srow = (sd.q_pos0 + r) % p.ring;
        const size_t src = ((static_cast<size_t>(seq) * p.rows + r) * p.kv_heads + h) * p.head_dim + v * VEC;
        const size_t dst = ((static_cast<size_t>(sd.slot) * p.kv_heads + h) * p.ring + srow) * p.head_dim + v * VEC;
        store_converted<F16, VEC>(p.k, dst, p.k_src + src);
        store_converted<F16, VEC>(p.v, dst, p.v_src + src);
    }
}

template <bool F16, int VEC>
__global__ void __launch_bounds__(256) convert_kernel(const float* src, void* dst, size_t n_vec) {
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n_vec;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x)
        store_converted<F16, VEC>(dst, idx * VEC, src + idx * VEC);
}

// Snapshot gather (to_snapshot = 1) and restore scatter (to_snapshot = 0) for
// up to 64 layers of one slot in one launch.  A snapshot layer block is the
// layer's visible rows in absolute-position order, `[rows][kv_heads][D]` for K
// then V (crates/itak-kv/src/snapshot.rs:247-302); the device rows live at
// position % ring, so the stored range maps to at most two storage runs
// (crates/wgpu-compute/src/session.rs:320-346) - here resolved per row.
// VB = bytes moved per access: 16 when a head row is a multiple of 16 bytes,
// else one element.  A work item is (layer, K or V, block of kCopyRows rows,
// head, vector): its index arithmetic is done once and kCopyRows loads are in
// flight per thread; lanes run over the vectors of a head row, so a warp
// reads and writes whole 256-byte head rows.
constexpr uint32_t kCopyRows = 8;

template <int VB>
struct CopyVec;
template <>
struct CopyVec<16> { using type = uint4; };
template <>
struct CopyVec<4> { using type = uint32_t; };
template <>
struct CopyVec<2> { using type = unsigned short; };

template <int VB>
__global__ void __launch_bounds__(256) snapshot_copy_kernel(const __grid_constant__ CopyLaunch p) {
    using V = typename CopyVec<VB>::type;
    const uint32_t row_units = p.head_dim * p.elem_bytes / VB;  // vectors per (row, head)
    const unsigned long long total_k = p.vec_prefix[p.n_layers];
    const unsigned long long row_bytes = static_cast<unsigned long long>(p.head_dim) * p.elem_bytes;
    for (unsigned long long idx = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
         idx < p.total_vec; idx += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const bool is_v = idx >= total_k;
        const unsigned long long j = is_v ? idx - total_k : idx;
        // layer with vec_prefix[l] <= j < vec_prefix[l + 1]
        uint32_t lo = 0, hi = p.n_layers;
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (p.vec_prefix[mid] <= j) lo = mid; else hi = mid;
        }
        const CopyLayer L = p.layer[lo];
        // a layer holds fewer than 2^32 work items (the launcher checks), so 32-bit divides suffice
        uint32_t w = static_cast<uint32_t>(j - p.vec_prefix[lo]);
        const uint32_t u = w % row_units;
        w /= row_units;
        const uint32_t h = w % p.kv_heads;
        const uint32_t r0 = (w / p.kv_heads) * kCopyRows;
        const uint32_t nr = min(kCopyRows, L.rows - r0);
        uint32_t srow = (L.first_pos + r0) % L.ring;
        unsigned char* slab = static_cast<unsigned char*>(is_v ? p.v_slab : p.k_slab) +
                              (L.slab_off + (static_cast<unsigned long long>(p.slot) * p.kv_heads + h) * L.ring * p.head_dim) *
                                  p.elem_bytes +
                              static_cast<unsigned long long>(u) * VB;
        unsigned char* snap = static_cast<unsigned char*>(p.snap) +
                              ((is_v ? L.snap_v : L.snap_k) +
                               (static_cast<unsigned long long>(r0) * p.kv_heads + h) * p.head_dim) * p.elem_bytes +
                              static_cast<unsigned long long>(u) * VB;
        const unsigned long long snap_step = row_bytes * p.kv_heads;
        V vals[kCopyRows];
        uint32_t srows[kCopyRows];
#pragma unroll
        for (uint32_t i = 0; i < kCopyRows; ++i) {
            srows[i] = srow;
            if (++srow == L.ring) srow = 0;
        }
        if (p.to_snapshot) {
#pragma unroll
            for (uint32_t i = 0; i < kCopyRows; ++i)
                if (i < nr) vals[i] = *reinterpret_cast<const V*>(slab + srows[i] * row_bytes);
#pragma unroll
            for (uint32_t i = 0; i < kCopyRows; ++i)
                if (i < nr) *reinterpret_cast<V*>(snap + i * snap_step) = vals[i];
        } else {
#pragma unroll
            for (uint32_t i = 0; i < kCopyRows; ++i)
                if (i < nr) vals[i] = *reinterpret_cast<const V*>(snap + i * snap_step);
#pragma unroll
            for (uint32_t i = 0; i < kCopyRows; ++i)
                if (i < nr) *reinterpret_cast<V*>(slab + srows[i] * row_bytes) = vals[i];
        }
    }
}

int grid_for(size_t work_items, int threads) {
    // Enough CTAs to fill 148 SMs several times over, never more than the work.
    const size_t want = (work_items + threads - 1) / threads;
    const size_t cap = 148 * 16;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

cudaError_t launch_append(const AppendLaunch& p, bool f16, cudaStream_t s, uint64_t* launches) {
    const bool vec = (p.head_dim % 8) == 0;
    const size_t items = static_cast<size_t>(p.n_seqs) * p.rows * p.kv_heads * (vec ? p.head_dim / 8 : p.head_dim);
    if (items == 0) return cudaSuccess;
    const int grid = grid_for(items, 256);
    if (f16 && vec) append_kernel<true, 8><<<grid, 256, 0, s>>>(p);
    else if (f16) append_kernel<true, 1><<<grid, 256, 0, s>>>(p);
    else if (vec) append_kernel<false, 8><<<grid, 256, 0, s>>>(p);
    else append_kernel<false, 1><<<grid, 256, 0, s>>>(p);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_convert(const float* src, void* dst, size_t n, bool f16, cudaStream_t s, uint64_t* launches) {
    if (n == 0) return cudaSuccess;
    const bool vec = (n % 8) == 0 && (reinterpret_cast<uintptr_t>(src) % 16) == 0 &&
                     (reinterpret_cast<uintptr_t>(dst) % 16) == 0;
    const size_t items = vec ? n / 8 : n;
    const int grid = grid_for(items, 256);
    if (f16 && vec) convert_kernel<true, 8><<<grid, 256, 0, s>>>(src, dst, items);
    else if (f16) convert_kernel<true, 1><<<grid, 256, 0, s>>>(src, dst, items);
    else if (vec) convert_kernel<false, 8><<<grid, 256, 0, s>>>(src, dst, items);
    else convert_kernel<false, 1><<<grid, 256, 0, s>>>(src, dst, items);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_snapshot_copy(const CopyLaunch& p, cudaStream_t s, uint64_t* launches) {
    if (p.total_vec == 0) return cudaSuccess;
    for (uint32_t l = 0; l < p.n_layers; ++l)
        if (p.vec_prefix[l + 1] - p.vec_prefix[l] > 0xffffffffull) return cudaErrorInvalidValue;
    const uint32_t row_bytes = p.head_dim * p.elem_bytes;
    const int grid = grid_for(p.total_vec, 256);
    if (row_bytes % 16 == 0) snapshot_copy_kernel<16><<<grid, 256, 0, s>>>(p);
    else if (p.elem_bytes == 4) snapshot_copy_kernel<4><<<grid, 256, 0, s>>>(p);
    else snapshot_copy_kernel<2><<<grid, 256, 0, s>>>(p);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk
