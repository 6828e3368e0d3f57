// Device helpers shared by the attention kernels: PTX wrappers and the CTA
// epilogue that turns per-split partial results into the final output.
#pragma once

#include "kernels.cuh"

namespace itk {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global -> shared copy that bypasses L1 (the cache is
// streamed once per step).  src_bytes == 0 writes 16 zero bytes and reads nothing.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr)
                 : "memory");
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col).
// Fragment ownership, with g = lane / 4 and t = lane % 4:
//   a[0] = A[g][2t..2t+1]      a[1] = A[g+8][2t..2t+1]
//   a[2] = A[g][2t+8..2t+9]    a[3] = A[g+8][2t+8..2t+9]
//   b0   = B[2t..2t+1][g]      b1   = B[2t+8..2t+9][g]
//   c[0..1] = D[g][2t..2t+1]   c[2..3] = D[g+8][2t..2t+1]
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi) {
    return static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
}

// x = hi + lo with hi = fp16(x) and lo = fp16(x - hi): two half operands that
// together carry ~22 bits of x.  An f16 tensor-core product against an exact
// f16 cache element then reproduces the f32 product to ~1e-7 relative.
__device__ __forceinline__ void split_half(float x, __half& hi, __half& lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}

constexpr float kLog2e = 1.4426950408889634f;

// Final-output stores: to AttnLaunch::out when set, and to every rank's gather buffer when the launch gathers.
__device__ __forceinline__ void store_out(const AttnLaunch& p, size_t off, float v) {
    if (p.out) p.out[off] = v;
    for (uint32_t j = 0; j < p.gather.n_peers; ++j) p.gather.peer_out[j][off] = v;
}
__device__ __forceinline__ void store_out4(const AttnLaunch& p, size_t off4, float4 v) {
    if (p.out) reinterpret_cast<float4*>(p.out)[off4] = v;
    for (uint32_t j = 0; j < p.gather.n_peers; ++j) reinterpret_cast<float4*>(p.gather.peer_out[j])[off4] = v;
}
// After a cell's output went out: make it visible system-wide, then count it on every rank (counter of the
// cell's sequence, `unit` = its index in the launch).
__device__ __forceinline__ void signal_cell_delivered(const AttnLaunch& p, uint32_t unit) {
    if (p.gather.n_peers == 0) return;
    // The CTA's stores are ordered before the barrier, and one thread's system-scope fence after it is cumulative
    // over them (the grid-barrier idiom): one fence per CTA instead of one per thread.  Then a reduction per peer
    // (no value comes back, so nothing waits for another NVLink round trip).
    __syncthreads();
    if (threadIdx.x == 0) {
        if (p.gather.local_only != 0)
            __threadfence();
        else
            __threadfence_system();
        ITK_TRACE(p, 15);  // (timeline build) the fence has returned
        for (uint32_t j = 0; j < p.gather.n_peers; ++j)
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;\n" ::"l"(p.gather.peer_flags[j] + unit * kMaxPeers + p.gather.my_rank) : "memory");
    }
}

constexpr uint32_t kFusedSumMinParts = 13;  // cells shared by more parts than one register batch take the fused sum
constexpr int kMaxSplits = 256;  // upper bound on the partials merged for one cell (sizes the merge scratch)

// The merge's per-part weights: reads the (max, sum) pairs of every part of a cell (all requested together), then
// w_m[part][head] = 2^(max_part - max_all) and inv_l[head] = 1 / sum of the weighted sums.  Ends with a CTA barrier.
template <int THREADS, int MAXP>
__device__ __forceinline__ void finish_weights(const float* all_ml, uint32_t n_parts, uint32_t nh, float* w_m, float* w_l,
                                               float* inv_l) {
    const uint32_t tid = threadIdx.x;
    {   // the (max, sum) pairs of every part, requested together (a fixed trip count keeps the loads independent)
        constexpr int kRounds = (MAXP * kHeadsPerCta + THREADS - 1) / THREADS;
        float2 ml[kRounds];
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const uint32_t i = tid + r * THREADS;
            ml[r] = make_float2(-INFINITY, 0.f);
            if (i < n_parts * kHeadsPerCta && i % kHeadsPerCta < nh)
                ml[r] = __ldcg(reinterpret_cast<const float2*>(all_ml) + i);
        }
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const uint32_t i = tid + r * THREADS;
            if (i < n_parts * kHeadsPerCta) {
                w_m[i] = ml[r].x;
                w_l[i] = ml[r].y;
            }
        }
    }
    __syncthreads();
    {   // per-head weights: sixteen lanes per head (every lane of the first 128 threads takes part in the shuffles)
        static_assert(THREADS >= 16 * kHeadsPerCta && THREADS % 32 == 0, "sixteen lanes per head");
        if (tid < 16 * kHeadsPerCta) {
            const uint32_t h = tid >> 4, q = tid & 15u;
            const bool live = h < nh;
            float M = -INFINITY;
            if (live)
                for (uint32_t s = q; s < n_parts; s += 16) M = fmaxf(M, w_m[s * kHeadsPerCta + h]);
#pragma unroll
            for (int d = 1; d < 16; d <<= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
            float L = 0.f;
            if (live)
                for (uint32_t s = q; s < n_parts; s += 16) {
                    const float ms = w_m[s * kHeadsPerCta + h];
                    const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
                    w_m[s * kHeadsPerCta + h] = w;
                    L += w * w_l[s * kHeadsPerCta + h];
                }
#pragma unroll
            for (int d = 1; d < 16; d <<= 1) L += __shfl_xor_sync(0xffffffffu, L, d);
            if (live && q == 0) inv_l[h] = 1.f / L;
        }
    }
    __syncthreads();
}


// CTA epilogue for one cell = (unit, head chunk).  On entry the CTA's own result
// for its part of the cell's key range sits in shared memory: fo[8][D]
// (unnormalised sum of p * v), fm[8] (running max, log2 domain, -inf when the
// part was empty) and fl[8] (sum of p).  `n_parts` CTAs share the cell and this
// one is number `part`.  With one part the output is written directly.
// Otherwise the partial goes to global scratch (p.splits slots per cell), the
// CTA takes a ticket, and the CTA that draws the last ticket merges every part
// (log-sum-exp) and writes the output; nobody waits.
// The merge's global loads are independent of each other: the (max, sum) pairs
// of every split (which become per-split weights in `wscratch`, shared memory,
// 2 * MAXP * 8 + 8 floats) and the first batch of partial outputs are requested
// together; every output channel is then a weighted sum over splits.
// With AttnLaunch::acc_o set, a cell shared by more than kFusedSumMinParts CTAs
// is summed in L2 instead (see below) and the last arrival reads one
// accumulator rather than every part.
// The ticket counter (and the accumulator) is left at zero for the next launch, before the cell is announced.
template <int THREADS, int MAXP>
__device__ __forceinline__ void finish_unit(const AttnLaunch& p, uint32_t unit, uint32_t hy, uint32_t n_parts,
                                            uint32_t part, uint32_t head0, uint32_t nh, uint32_t D, const float* fo,
                                            const float* fm, const float* fl, int* s_flag, float* wscratch) {
    const uint32_t tid = threadIdx.x;
    const uint32_t HY = p.layer.kv_heads * p.gchunks;
    const size_t out_off = (static_cast<size_t>(unit) * p.q_heads + head0) * D;  // element offset of the cell's rows
    if (n_parts == 1) {
        for (uint32_t idx = tid; idx < nh * D; idx += THREADS) {
            const uint32_t h = idx / D;
            store_out(p, out_off + idx, fo[idx] / fl[h]);
        }
        signal_cell_delivered(p, unit);
        return;
    }
    const size_t cell = static_cast<size_t>(unit) * HY + hy;
    float* po = p.part_o + (cell * p.splits + part) * (kHeadsPerCta * D);
    float* pml = p.part_ml + (cell * p.splits + part) * (kHeadsPerCta * 2);
    for (uint32_t idx = tid; idx < nh * D; idx += THREADS) po[idx] = fo[idx];
    if (tid < nh) {
        pml[2 * tid] = fm[tid];
        pml[2 * tid + 1] = fl[tid];
    }
    // A cell shared by many CTAs is not merged by reading every part back: each part also adds its output, scaled
    // by 2^max of the part, into one accumulator per cell with reductions performed in L2, and the last arrival
    // only reads that sum.  Sums of terms scaled by their own maxima are as good as sums scaled by the common
    // maximum while every factor stays far inside the f32 range; a part whose maximum lies outside
    // [-kAccRange, kAccRange] (log2 domain) raises the cell's flag instead and the merge below takes the exact path
    // over the stored parts.  The order of the additions varies from launch to launch, so results on this path agree
    // to rounding, not bit for bit.
    constexpr float kAccRange = 60.f;
    const bool fused_sum = p.acc_o != nullptr && n_parts > kFusedSumMinParts && (D & 3u) == 0 && nh * D / 4 <= 2 * THREADS;
    if (fused_sum) {
        bool in_range = true;
        for (uint32_t h = 0; h < nh; ++h) in_range = in_range && (fm[h] == -INFINITY || fabsf(fm[h]) <= kAccRange);
        if (in_range) {
            // four channels per reduction: the accumulator's lines are hammered by every CTA of the cell at about
            // the same time, and L2 performs same-address reductions one after another
            float* ao = p.acc_o + cell * (kHeadsPerCta * D);
            for (uint32_t idx4 = tid; idx4 < nh * D / 4; idx4 += THREADS) {
                const float m = fm[(idx4 * 4) / D];
                if (m != -INFINITY) {
                    const float w = fast_exp2(m);
                    const float4 v = *reinterpret_cast<const float4*>(fo + idx4 * 4);
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(ao + idx4 * 4), "f"(v.x * w), "f"(v.y * w),
                                 "f"(v.z * w), "f"(v.w * w)
                                 : "memory");
                }
            }
            if (tid < nh && fm[tid] != -INFINITY) atomicAdd(p.acc_l + cell * kHeadsPerCta + tid, fl[tid] * fast_exp2(fm[tid]));
        } else if (tid == 0) {
            atomicOr(p.acc_flag + cell, 1u);
        }
    }
    __syncthreads();
    ITK_TRACE(p, 8);
    if (tid == 0) {
        __threadfence();  // cumulative over the CTA's stores and reductions above (ordered before the barrier)
        const unsigned int ticket = atomicAdd(p.tickets + cell, 1u);
        *s_flag = (ticket == n_parts - 1) ? 1 : 0;
    }
    __syncthreads();
    ITK_TRACE(p, 9);
    if (*s_flag == 0) return;
    ITK_TRACE(p, 6);  // this CTA drew the last ticket of a cell and merges it
    __threadfence();
    if (fused_sum) {
        float* ao = p.acc_o + cell * (kHeadsPerCta * D);
        float* al = p.acc_l + cell * kHeadsPerCta;
        const unsigned int slow = __ldcg(p.acc_flag + cell);
        {
            const uint32_t cols = nh * D / 4, c0 = tid, c1 = tid + THREADS;
            float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
            float l0 = 1.f, l1 = 1.f;
            if (c0 < cols) {
                a0 = __ldcg(reinterpret_cast<const float4*>(ao) + c0);
                l0 = __ldcg(al + (c0 * 4) / D);
            }
            if (c1 < cols) {
                a1 = __ldcg(reinterpret_cast<const float4*>(ao) + c1);
                l1 = __ldcg(al + (c1 * 4) / D);
            }
            __syncthreads();  // every thread holds its share: the accumulators can be cleared for the next launch
            ITK_TRACE(p, 10);
            const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c0 < cols) reinterpret_cast<float4*>(ao)[c0] = zero;
            if (c1 < cols) reinterpret_cast<float4*>(ao)[c1] = zero;
            if (tid < kHeadsPerCta) al[tid] = 0.f;
            if (tid == 0) p.acc_flag[cell] = 0u;
            if (slow == 0u) {
                const float i0 = 1.f / l0, i1 = 1.f / l1;
                if (c0 < cols) store_out4(p, out_off / 4 + c0, make_float4(a0.x * i0, a0.y * i0, a0.z * i0, a0.w * i0));
                if (c1 < cols) store_out4(p, out_off / 4 + c1, make_float4(a1.x * i1, a1.y * i1, a1.z * i1, a1.w * i1));
                ITK_TRACE(p, 11);
                // the counter is back at zero BEFORE the cell is announced: a launch that orders itself by the
                // arrival counters alone may take its first ticket the moment it sees the announcement
                if (tid == 0) p.tickets[cell] = 0u;
                signal_cell_delivered(p, unit);
                return;
            }
        }
    }
    const float* all_o = p.part_o + cell * p.splits * (kHeadsPerCta * D);
    const float* all_ml = p.part_ml + cell * p.splits * (kHeadsPerCta * 2);
    float* w_m = wscratch;                        // [splits][8] maxima, then weights
    float* w_l = wscratch + MAXP * kHeadsPerCta;  // [parts][8] sums
    float* inv_l = w_l + MAXP * kHeadsPerCta;     // [8]
    // Vector path: a thread owns up to two float4 columns and keeps kBatch parts x 2 columns of loads in flight.
    // The partial outputs do not depend on the weights, so the first batch is requested together with the
    // (max, sum) pairs: merging a cell that dozens of CTAs shared costs two or three memory round trips.
    constexpr int kBatch = 13;
    const bool vec = (D & 3u) == 0;
    const uint32_t cols = nh * D / 4;
    const size_t pstride = kHeadsPerCta * D / 4;  // float4s per part
    const float4* src4 = reinterpret_cast<const float4*>(all_o);
    uint32_t c0 = tid, c1 = tid + THREADS;
    bool one = vec && c0 < cols, two = vec && c1 < cols;
    float4 v0[kBatch], v1[kBatch];
    auto load_batch = [&](uint32_t s) {
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            const uint32_t si = s + i < n_parts ? s + i : s;  // clamped; its weight is zeroed below
            v0[i] = one ? __ldcg(src4 + si * pstride + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
            v1[i] = two ? __ldcg(src4 + si * pstride + c1) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    if (vec) load_batch(0);
    finish_weights<THREADS, MAXP>(all_ml, n_parts, nh, w_m, w_l, inv_l);
    ITK_TRACE(p, 11);
    for (uint32_t base = 0; vec && base < cols; base += 2 * THREADS) {  // one round unless nh * D > 8 * THREADS
        if (base != 0) {
            c0 = base + tid;
            c1 = c0 + THREADS;
            one = c0 < cols;
            two = c1 < cols;
        }
        const uint32_t h0 = one ? (c0 * 4) / D : 0u, h1 = two ? (c1 * 4) / D : h0;
        float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
        for (uint32_t s = 0; s < n_parts; s += kBatch) {
            if (s != 0 || base != 0) load_batch(s);
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const bool ok = s + i < n_parts;
                const float w0 = ok ? w_m[(s + i) * kHeadsPerCta + h0] : 0.f;
                const float w1 = ok ? w_m[(s + i) * kHeadsPerCta + h1] : 0.f;
                a0.x += w0 * v0[i].x; a0.y += w0 * v0[i].y; a0.z += w0 * v0[i].z; a0.w += w0 * v0[i].w;
                a1.x += w1 * v1[i].x; a1.y += w1 * v1[i].y; a1.z += w1 * v1[i].z; a1.w += w1 * v1[i].w;
            }
        }
        ITK_TRACE(p, 12);
        const float i0 = inv_l[h0], i1 = inv_l[h1];
        if (one) store_out4(p, out_off / 4 + c0, make_float4(a0.x * i0, a0.y * i0, a0.z * i0, a0.w * i0));
        if (two) store_out4(p, out_off / 4 + c1, make_float4(a1.x * i1, a1.y * i1, a1.z * i1, a1.w * i1));
    }
    if (!vec) {
        for (uint32_t idx = tid; idx < nh * D; idx += THREADS) {
            const uint32_t h = idx / D;
            const float* src = all_o + idx;
            float acc = 0.f;
            for (uint32_t s = 0; s < n_parts; ++s)
                acc += w_m[s * kHeadsPerCta + h] * __ldcg(src + static_cast<size_t>(s) * (kHeadsPerCta * D));
            store_out(p, out_off + idx, acc * inv_l[h]);
        }
    }
    if (tid == 0) p.tickets[cell] = 0u;  // before the announcement, as above
    signal_cell_delivered(p, unit);
}

}  // namespace itk
