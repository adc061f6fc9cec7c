// Memory-bound kernels around the matrix products: embedding rows into the
// fp32 residual stream, residual add fused with RMSNorm, bias + rotary position
// encoding fused with the write of K and V into cache pages, SiLU(gate)*up.
//
// All statistics, angles and sums are fp32; `T` is the storage type of
// activations and cache (float or bf16).  Every kernel takes any row width.
#include "common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

// ---------------------------------------------------------------------------
// Embedding: resid[n, :] = float(table[ids[n], :]) * scale (fp32 product; scale 1 for the reference's
// model, flow_engine/model.py:176).  An id below zero names a token that is still on the
// device: -(i + 1) stands for device_tokens[i], the i-th token the previous step sampled, so a
// step can be launched before the host has seen its input tokens.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(float* __restrict__ resid, const T* __restrict__ table,
                             const int* __restrict__ ids, const int* __restrict__ device_tokens, int n_device_tokens,
                             int hidden, int vocab, float scale, int* status) {
    TW_TIMELINE_SCOPE(TW_K_EMBED);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 && device_tokens && -(id + 1) < n_device_tokens) id = device_tokens[-(id + 1)];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, TW_ERR_TOKEN_ID);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) resid[(size_t)n * hidden + i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    float* dst = resid + (size_t)n * hidden;
    if constexpr (sizeof(T) == 2) {
        // 16 bytes per load where the row allows: a decode step waits for this kernel's one round trip to memory
        if ((hidden & 7) == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0) {
            for (int i = threadIdx.x; i < (hidden >> 3); i += blockDim.x) {
                const uint4 raw = reinterpret_cast<const uint4*>(row)[i];
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
                const float2 c = __bfloat1622float2(h2[2]), d = __bfloat1622float2(h2[3]);
                reinterpret_cast<float4*>(dst)[2 * i] = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
                reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(c.x * scale, c.y * scale, d.x * scale, d.y * scale);
            }
            return;
        }
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = tw_to_float(row[i]) * scale;
}

TW_EXPORT int tw_embed(void* resid, const void* table, const int* ids, const int* device_tokens, int n_device_tokens,
                       int n_tokens, int hidden, int vocab, float scale, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dtype == TW_F32)
        tw_launch(embed_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, 1, (float*)resid, (const float*)table, ids, device_tokens, n_device_tokens, hidden, vocab, scale, status);
    else
        tw_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, 1, (float*)resid, (const __nv_bfloat16*)table, ids,
                                                                   device_tokens, n_device_tokens, hidden, vocab, scale, status);
    return TW_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm.
//   v = resid[src] + delta_scale * delta[src]     (delta may be null; the product and the sum are fp32)
//   resid[src] = v                         (only when rows == null)
//   out[r] = T( (v * (1 / sqrt(mean(v^2) + eps))) * weight )
// rows != null selects source rows (the final norm runs on the wanted rows
// only); the residual stream is then left untouched.
// Reference: flow_engine/model.py:21-23 (fp32 statistics).  The reference casts
// the normalised value to the activation type before the multiply by the
// weight; here the product is formed in fp32 and rounded once.
// ---------------------------------------------------------------------------
// The delta is either a dense tensor of the activation type or `nsplit` fp32 slices of a
// split matrix product ([slice][row][hidden], slices `split_stride` floats apart), which
// are added here in slice order.
#define TW_NORM_THREADS 512
#define TW_NORM_MAXV 16          // values a thread keeps in registers: rows up to 512 * 16 wide take the one-pass path

template <typename T, bool ONE_PASS>
__global__ void __launch_bounds__(TW_NORM_THREADS)
add_rmsnorm_kernel(T* __restrict__ out, float* __restrict__ resid, const T* __restrict__ delta,
                   const float* __restrict__ partial, int nsplit, size_t split_stride,
                   const float* __restrict__ weight, float eps, int hidden, const int* __restrict__ rows, float dscale) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    TW_TIMELINE_SCOPE(TW_K_NORM);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int src = rows ? rows[r] : r;
    float* x = resid + (size_t)src * hidden;
    const T* d = delta ? delta + (size_t)src * hidden : nullptr;
    const float* ps = partial ? partial + (size_t)src * hidden : nullptr;
    const bool has_delta = d || ps;
    auto delta_at = [&](int i) -> float {
        if (d) return tw_to_float(d[i]) * dscale;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;      // fixed order: ((s0 + s1) + (s2 + s3)) over interleaved slices
        int k = 0;
        for (; k + 4 <= nsplit; k += 4) {
            s0 += ps[(size_t)k * split_stride + i];
            s1 += ps[(size_t)(k + 1) * split_stride + i];
            s2 += ps[(size_t)(k + 2) * split_stride + i];
            s3 += ps[(size_t)(k + 3) * split_stride + i];
        }
        for (; k < nsplit; ++k) s0 += ps[(size_t)k * split_stride + i];
        return ((s0 + s1) + (s2 + s3)) * dscale;
    };
    T* o = out + (size_t)r * hidden;
    if (ONE_PASS) {
        float v[TW_NORM_MAXV];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int i = threadIdx.x + j * TW_NORM_THREADS;
            v[j] = 0.f;
            if (i < hidden) {
                v[j] = x[i];
                if (has_delta) v[j] += delta_at(i);
                if (!rows && has_delta) x[i] = v[j];
                ss += v[j] * v[j];
            }
        }
        ss = tw_block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int i = threadIdx.x + j * TW_NORM_THREADS;
            if (i < hidden) o[i] = tw_from_float<T>((v[j] * inv) * weight[i]);
        }
    } else {
        float ss = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = x[i];
            if (has_delta) v += delta_at(i);
            if (!rows && has_delta) x[i] = v;
            ss += v * v;
        }
        ss = tw_block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = x[i];
            if (rows && has_delta) v += delta_at(i);
            o[i] = tw_from_float<T>((v * inv) * weight[i]);
        }
    }
}

// The same for steps with few rows: a cluster of CTAs shares one row, each CTA owning a
// range of columns, and the partial sums of squares meet in distributed shared memory
// (added in rank order, so the result does not depend on timing).  With one CTA per row a
// decode step of 8 rows would keep only 8 SMs busy.
#define TW_NORM_CLUSTER 8
#define TW_NORM_CTHREADS 256
#define TW_NORM_CMAXV 4

template <typename T>
__global__ void __launch_bounds__(TW_NORM_CTHREADS)
add_rmsnorm_cluster_kernel(T* __restrict__ out, float* __restrict__ resid, const T* __restrict__ delta,
                           const float* __restrict__ partial, int nsplit, size_t split_stride,
                           const float* __restrict__ weight, float eps, int hidden, const int* __restrict__ rows, float dscale) {
    __shared__ float scratch[33];
    __shared__ float all_ss[TW_NORM_CLUSTER];      // every block's sum of squares, written here by the blocks themselves
    TW_TIMELINE_SCOPE(TW_K_NORM_CLUSTER);
    // What no kernel of the step writes (the row indices, the norm's weights) is read before the wait for the
    // kernel before this one: this kernel is a chain of round trips, and these two need not be in it.
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int r = blockIdx.x / TW_NORM_CLUSTER;
    const int src = rows ? rows[r] : r;
    const int chunk = (hidden + TW_NORM_CLUSTER - 1) / TW_NORM_CLUSTER;
    const int c0 = rank * chunk, c1 = min(hidden, c0 + chunk);
    float wv[TW_NORM_CMAXV];
#pragma unroll
    for (int j = 0; j < TW_NORM_CMAXV; ++j) {
        const int i = c0 + threadIdx.x + j * TW_NORM_CTHREADS;
        wv[j] = i < c1 ? weight[i] : 0.f;
    }
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_launch_dependents_now();     // 64 small blocks: the product that follows may settle on the SMs meanwhile (1 % of a decode step)
    float* x = resid + (size_t)src * hidden;
    const T* d = delta ? delta + (size_t)src * hidden : nullptr;
    const float* ps = partial ? partial + (size_t)src * hidden : nullptr;
    const bool has_delta = d || ps;
    float v[TW_NORM_CMAXV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < TW_NORM_CMAXV; ++j) {
        const int i = c0 + threadIdx.x + j * TW_NORM_CTHREADS;
        v[j] = 0.f;
        if (i < c1) {
            float dv = 0.f;
            if (d) {
                dv = tw_to_float(d[i]);
            } else if (ps) {
                // The slices are summed in the order every consumer of a split product uses: whole groups of
                // four into four sums by k mod 4, the rest into the first, then (s0 + s1) + (s2 + s3).  The
                // first sixteen are loaded before anything is added, so that they are one round trip to L2
                // and not one per group (this kernel is nothing but latency).
                float t[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) t[u] = u < nsplit ? ps[(size_t)u * split_stride + i] : 0.f;
                const int full = nsplit & ~3;
                float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    if (u < full) sum[u & 3] += t[u];
                }
                int k = 16;
                for (; k + 4 <= nsplit; k += 4) {
                    sum[0] += ps[(size_t)k * split_stride + i];
                    sum[1] += ps[(size_t)(k + 1) * split_stride + i];
                    sum[2] += ps[(size_t)(k + 2) * split_stride + i];
                    sum[3] += ps[(size_t)(k + 3) * split_stride + i];
                }
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    if (u >= full && u < nsplit) sum[0] += t[u];
                }
                for (k = max(k, full); k < nsplit; ++k) sum[0] += ps[(size_t)k * split_stride + i];
                dv = (sum[0] + sum[1]) + (sum[2] + sum[3]);
            }
            v[j] = x[i] + dv * dscale;
            if (!rows && has_delta) x[i] = v[j];
            ss += v[j] * v[j];
        }
    }
    ss = tw_block_sum(ss, scratch);
    // every block hands its sum to all blocks of the cluster (one remote store each), so that after one
    // cluster barrier each block finds the eight sums in its own shared memory and nobody reads a neighbour's
    if (threadIdx.x < TW_NORM_CLUSTER) *cluster.map_shared_rank(&all_ss[rank], threadIdx.x) = ss;
    cluster.sync();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < TW_NORM_CLUSTER; ++k) total += all_ss[k];       // in rank order
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    T* o = out + (size_t)r * hidden;
#pragma unroll
    for (int j = 0; j < TW_NORM_CMAXV; ++j) {
        const int i = c0 + threadIdx.x + j * TW_NORM_CTHREADS;
        if (i < c1) o[i] = tw_from_float<T>((v[j] * inv) * wv[j]);
    }
}

__device__ __forceinline__ float4 tw_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 tw_load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void tw_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void tw_store4(__nv_bfloat16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}

// Many rows (prompt portions): four values per thread and access, one pass, values kept in registers.
// Dense delta only; hidden a multiple of 4 and at most 4 * 256 * V4 wide.  V4 = float4 per thread: 4 for rows up
// to 4,096 wide (half the registers, twice the blocks per SM), 8 up to 8,192.
#define TW_NORM_V4 8
template <typename T, int V4>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec4_kernel(T* __restrict__ out, float* __restrict__ resid, const T* __restrict__ delta,
                        const float* __restrict__ weight, float eps, int hidden, const int* __restrict__ rows, float dscale) {
    __shared__ float scratch[33];
    TW_TIMELINE_SCOPE(TW_K_NORM);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float4* x4 = reinterpret_cast<float4*>(resid + (size_t)src * hidden);
    const int n4 = hidden >> 2;
    float4 v[V4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < V4; ++j) {
        const int i = threadIdx.x + j * 256;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            v[j] = x4[i];
            if (delta) {
                const float4 d = tw_load4(delta + (size_t)src * hidden + 4 * i);
                v[j].x += d.x * dscale; v[j].y += d.y * dscale; v[j].z += d.z * dscale; v[j].w += d.w * dscale;
                if (!rows) x4[i] = v[j];
            }
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    ss = tw_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    const float4* w4 = reinterpret_cast<const float4*>(weight);
#pragma unroll
    for (int j = 0; j < V4; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 w = w4[i];
            tw_store4(out + (size_t)r * hidden + 4 * i,
                      make_float4((v[j].x * inv) * w.x, (v[j].y * inv) * w.y, (v[j].z * inv) * w.z, (v[j].w * inv) * w.w));
        }
    }
}

template <typename T>
static int launch_add_rmsnorm(T* out, float* resid, const T* delta, const float* partial, int nsplit,
                              size_t split_stride, const float* weight, float eps, int n_rows, int hidden,
                              const int* rows, float dscale, cudaStream_t stream) {
    if (n_rows <= 64 && hidden >= 1024 && hidden <= TW_NORM_CLUSTER * TW_NORM_CTHREADS * TW_NORM_CMAXV) {
        return tw_launch(add_rmsnorm_cluster_kernel<T>, dim3(n_rows * TW_NORM_CLUSTER), dim3(TW_NORM_CTHREADS), 0, stream,
                         TW_NORM_CLUSTER, out, resid, delta, partial, nsplit, split_stride, weight, eps, hidden, rows, dscale);
    }
    if (!partial && (hidden & 3) == 0 && hidden <= 4 * 256 * TW_NORM_V4) {
        if (hidden <= 4 * 256 * 4)
            tw_launch(add_rmsnorm_vec4_kernel<T, 4>, dim3(n_rows), dim3(256), 0, stream, 1, out, resid, delta, weight, eps,
                      hidden, rows, dscale);
        else
            tw_launch(add_rmsnorm_vec4_kernel<T, TW_NORM_V4>, dim3(n_rows), dim3(256), 0, stream, 1, out, resid, delta, weight,
                      eps, hidden, rows, dscale);
        return TW_LAUNCH_CHECK();
    }
    if (hidden <= TW_NORM_THREADS * TW_NORM_MAXV)
        tw_launch(add_rmsnorm_kernel<T, true>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, out, resid, delta, partial, nsplit,
                                                                            split_stride, weight, eps, hidden, rows, dscale);
    else
        tw_launch(add_rmsnorm_kernel<T, false>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, out, resid, delta, partial, nsplit,
                                                                             split_stride, weight, eps, hidden, rows, dscale);
    return TW_LAUNCH_CHECK();
}

TW_EXPORT int tw_add_rmsnorm(void* out, float* resid, const void* delta, const float* partial, int nsplit,
                             long split_stride, const float* weight, float eps, int n_rows, int hidden,
                             const int* rows, float delta_scale, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (delta && partial) return (int)cudaErrorInvalidValue;
    if (dtype == TW_F32)
        return launch_add_rmsnorm<float>((float*)out, resid, (const float*)delta, partial, nsplit, (size_t)split_stride,
                                         weight, eps, n_rows, hidden, rows, delta_scale, stream);
    return launch_add_rmsnorm<__nv_bfloat16>((__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, partial, nsplit,
                                             (size_t)split_stride, weight, eps, n_rows, hidden, rows, delta_scale, stream);
}

// ---------------------------------------------------------------------------
// RMSNorm of a sub-layer's OUTPUT, added to the residual stream (a block that normalises what a
// sub-layer returns instead of what it reads):
//   y = delta[r]                            (a tensor of the activation type, or fp32 slices added in slice order)
//   resid[r] += (y * (1 / sqrt(mean(y^2) + eps))) * weight          all in fp32
//   copy[r] = T(resid[r])                   (copy may be null: the rows the next sub-layer reads, in its type)
// ---------------------------------------------------------------------------
template <typename T, bool ONE_PASS>
__global__ void __launch_bounds__(TW_NORM_THREADS)
rmsnorm_to_residual_kernel(float* __restrict__ resid, T* __restrict__ copy, const T* __restrict__ delta,
                           const float* __restrict__ partial, int nsplit, size_t split_stride,
                           const float* __restrict__ weight, float eps, int hidden) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    TW_TIMELINE_SCOPE(TW_K_NORM);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    float* x = resid + (size_t)r * hidden;
    const T* d = delta ? delta + (size_t)r * hidden : nullptr;
    const float* ps = partial ? partial + (size_t)r * hidden : nullptr;
    auto delta_at = [&](int i) -> float {
        if (d) return tw_to_float(d[i]);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;      // the order every consumer of a split product uses
        int k = 0;
        for (; k + 4 <= nsplit; k += 4) {
            s0 += ps[(size_t)k * split_stride + i];
            s1 += ps[(size_t)(k + 1) * split_stride + i];
            s2 += ps[(size_t)(k + 2) * split_stride + i];
            s3 += ps[(size_t)(k + 3) * split_stride + i];
        }
        for (; k < nsplit; ++k) s0 += ps[(size_t)k * split_stride + i];
        return (s0 + s1) + (s2 + s3);
    };
    T* c = copy ? copy + (size_t)r * hidden : nullptr;
    if (ONE_PASS) {
        float v[TW_NORM_MAXV];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int i = threadIdx.x + j * TW_NORM_THREADS;
            v[j] = i < hidden ? delta_at(i) : 0.f;
            ss += v[j] * v[j];
        }
        ss = tw_block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int i = threadIdx.x + j * TW_NORM_THREADS;
            if (i < hidden) {
                const float nv = x[i] + (v[j] * inv) * weight[i];
                x[i] = nv;
                if (c) c[i] = tw_from_float<T>(nv);
            }
        }
    } else {
        float ss = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = delta_at(i);
            ss += v * v;
        }
        ss = tw_block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float nv = x[i] + (delta_at(i) * inv) * weight[i];
            x[i] = nv;
            if (c) c[i] = tw_from_float<T>(nv);
        }
    }
}

// The same with four values per access (dense delta, width a multiple of 4 and at most 4 * 256 * V4).
template <typename T, int V4>
__global__ void __launch_bounds__(256)
rmsnorm_to_residual_vec4_kernel(float* __restrict__ resid, T* __restrict__ copy, const T* __restrict__ delta,
                                const float* __restrict__ weight, float eps, int hidden) {
    __shared__ float scratch[33];
    TW_TIMELINE_SCOPE(TW_K_NORM);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int r = blockIdx.x;
    float4* x4 = reinterpret_cast<float4*>(resid + (size_t)r * hidden);
    const int n4 = hidden >> 2;
    float4 v[V4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < V4; ++j) {
        const int i = threadIdx.x + j * 256;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            v[j] = tw_load4(delta + (size_t)r * hidden + 4 * i);
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    ss = tw_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    const float4* w4 = reinterpret_cast<const float4*>(weight);
#pragma unroll
    for (int j = 0; j < V4; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 w = w4[i];
            float4 x = x4[i];
            x.x += (v[j].x * inv) * w.x; x.y += (v[j].y * inv) * w.y; x.z += (v[j].z * inv) * w.z; x.w += (v[j].w * inv) * w.w;
            x4[i] = x;
            if (copy) tw_store4(copy + (size_t)r * hidden + 4 * i, x);
        }
    }
}

template <typename T>
static int launch_rmsnorm_to_residual(float* resid, T* copy, const T* delta, const float* partial, int nsplit,
                                      size_t split_stride, const float* weight, float eps, int n_rows, int hidden,
                                      cudaStream_t stream) {
    if (!partial && (hidden & 3) == 0 && hidden <= 4 * 256 * TW_NORM_V4) {
        if (hidden <= 4 * 256 * 4)
            return tw_launch(rmsnorm_to_residual_vec4_kernel<T, 4>, dim3(n_rows), dim3(256), 0, stream, 1, resid, copy, delta,
                             weight, eps, hidden);
        return tw_launch(rmsnorm_to_residual_vec4_kernel<T, TW_NORM_V4>, dim3(n_rows), dim3(256), 0, stream, 1, resid, copy,
                         delta, weight, eps, hidden);
    }
    if (hidden <= TW_NORM_THREADS * TW_NORM_MAXV)
        return tw_launch(rmsnorm_to_residual_kernel<T, true>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, resid, copy,
                         delta, partial, nsplit, split_stride, weight, eps, hidden);
    return tw_launch(rmsnorm_to_residual_kernel<T, false>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, resid, copy,
                     delta, partial, nsplit, split_stride, weight, eps, hidden);
}

TW_EXPORT int tw_rmsnorm_to_residual(float* resid, void* copy, const void* delta, const float* partial, int nsplit,
                                     long split_stride, const float* weight, float eps, int n_rows, int hidden,
                                     int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!delta == !partial) return (int)cudaErrorInvalidValue;      // exactly one source
    if (dtype == TW_F32)
        return launch_rmsnorm_to_residual<float>(resid, (float*)copy, (const float*)delta, partial, nsplit,
                                                 (size_t)split_stride, weight, eps, n_rows, hidden, stream);
    return launch_rmsnorm_to_residual<__nv_bfloat16>(resid, (__nv_bfloat16*)copy, (const __nv_bfloat16*)delta, partial,
                                                     nsplit, (size_t)split_stride, weight, eps, n_rows, hidden, stream);
}

// out[i] = T(resid[i]): the fp32 residual rows in the type the matrix products read.
template <typename T>
__global__ void round_rows_kernel(T* __restrict__ out, const float* __restrict__ resid, long total) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = tw_from_float<T>(resid[i]);
}

TW_EXPORT int tw_round_rows(void* out, const float* resid, long total, int dtype, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == TW_F32)
        return tw_launch(round_rows_kernel<float>, dim3(blocks), dim3(threads), 0, stream, 1, (float*)out, resid, total);
    return tw_launch(round_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, resid,
                     total);
}

// ---------------------------------------------------------------------------
// Bias + rotary position encoding + cache write, one block per token.
//
// qkv row layout: [q heads | k heads | v heads], each head `D` wide.
//   x += bias                                       (bias may be null)
//   angle_i = float(position) * inv_freq[i]         (fp32; inv_freq may be null: no rotation)
//   y[i]        = x[i] * cos - x[i + D/2] * sin     (rotate-half pairing)
//   y[i + D/2]  = x[i + D/2] * cos + x[i] * sin
// q is rewritten in place; rotated k and v go to the page that the request's
// block table names for this position:
//   page = table[slot_row][pos / P];  element ((page * Hkv + h) * P + pos % P) * D + d
// Reference: flow_engine/model.py:26-33,184-187; flow_engine/cache.py:93-100.
// ---------------------------------------------------------------------------
// The source of a row is the qkv buffer itself or, when the projection was split over k,
// the sum of `nsplit` fp32 slices [slice][token][width]; q always lands in the qkv buffer.
#define TW_ROPE_THREADS 128

template <typename T>
__global__ void __launch_bounds__(TW_ROPE_THREADS)
rope_kv_write_kernel(T* __restrict__ qkv, int qkv_stride, const float* __restrict__ partial, int nsplit,
                     size_t split_stride, const float* __restrict__ bias, const int* __restrict__ positions,
                     const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot,
                     const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq,
                     T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hkv, int D, int page_size,
                     int num_pages, int write_cache, int* status) {
    TW_TIMELINE_SCOPE(TW_K_ROPE);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;  // padding row of a fixed-size batch
    const int pos = positions[n];
    const int half = D >> 1;
    T* row = qkv + (size_t)n * qkv_stride;
    const int width = (Hq + 2 * Hkv) * D;
    const float* prow = partial ? partial + (size_t)n * width : nullptr;
    auto src_at = [&](int col) -> float {
        if (!prow) return tw_to_float(row[col]);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int k = 0;
        for (; k + 4 <= nsplit; k += 4) {
            s0 += prow[(size_t)k * split_stride + col];
            s1 += prow[(size_t)(k + 1) * split_stride + col];
            s2 += prow[(size_t)(k + 2) * split_stride + col];
            s3 += prow[(size_t)(k + 3) * split_stride + col];
        }
        for (; k < nsplit; ++k) s0 += prow[(size_t)k * split_stride + col];
        return (s0 + s1) + (s2 + s3);
    };

    int page = -1;
    if (write_cache) {
        const int blk = pos / page_size;
        page = blk < table_stride ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, TW_ERR_PAGE);
            page = -1;
        }
    }
    const int in_page = pos % page_size;
    const int rot_pairs = (write_cache ? Hq + Hkv : Hq) * half;     // rotated (q, then k) pairs
    const int v_pairs = write_cache ? Hkv * half : 0;               // v is copied pair-wise, unrotated
    const int idx = blockIdx.y * TW_ROPE_THREADS + threadIdx.x;
    if (idx < rot_pairs) {
        const int head = idx / half, i = idx - head * half;
        const int col = head * D + i;
        float x1 = src_at(col), x2 = src_at(col + half);
        if (bias) { x1 += bias[col]; x2 += bias[col + half]; }
        float y1 = x1, y2 = x2;
        if (inv_freq) {
            const float ang = (float)pos * inv_freq[i];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            y1 = x1 * cs - x2 * sn;
            y2 = x2 * cs + x1 * sn;
        }
        if (head < Hq) {
            row[col] = tw_from_float<T>(y1);
            row[col + half] = tw_from_float<T>(y2);
        } else if (page >= 0) {
            const int kvh = head - Hq;
            T* dst = k_cache + (((size_t)page * Hkv + kvh) * page_size + in_page) * D;
            dst[i] = tw_from_float<T>(y1);
            dst[i + half] = tw_from_float<T>(y2);
        }
    } else if (idx < rot_pairs + v_pairs && page >= 0) {
        const int j = idx - rot_pairs;
        const int kvh = j / half, i = j - kvh * half;
        const int col = (Hq + Hkv) * D + kvh * D + i;
        float v1 = src_at(col), v2 = src_at(col + half);
        if (bias) { v1 += bias[col]; v2 += bias[col + half]; }
        T* dst = v_cache + (((size_t)page * Hkv + kvh) * page_size + in_page) * D;
        dst[i] = tw_from_float<T>(v1);
        dst[i + half] = tw_from_float<T>(v2);
    }
}

// bf16, dense source, head size a multiple of 16: a thread rotates eight neighbouring pairs with 16-byte accesses
// (or copies sixteen values of v).  Same arithmetic as the kernel above.
__global__ void __launch_bounds__(TW_ROPE_THREADS)
rope_kv_write_bf16x8_kernel(__nv_bfloat16* __restrict__ qkv, int qkv_stride, const float* __restrict__ bias,
                            const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ seq_slot, const int* __restrict__ block_table, int table_stride,
                            const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ k_cache,
                            __nv_bfloat16* __restrict__ v_cache, int Hq, int Hkv, int D, int page_size, int num_pages,
                            int write_cache, int* status) {
    TW_TIMELINE_SCOPE(TW_K_ROPE);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;
    const int pos = positions[n];
    const int half = D >> 1, groups = half >> 3;           // groups of 8 pairs per head
    __nv_bfloat16* row = qkv + (size_t)n * qkv_stride;
    int page = -1;
    if (write_cache) {
        const int blk = pos / page_size;
        page = blk < table_stride ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, TW_ERR_PAGE);
            page = -1;
        }
    }
    const int in_page = pos % page_size;
    // the angles depend on the position and the pair only: each is evaluated once per block, not once per head
    __shared__ float s_cos[128], s_sin[128];
    if (inv_freq) {
        for (int i = threadIdx.x; i < half; i += TW_ROPE_THREADS) sincosf((float)pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    __syncthreads();
    const int rot_items = (write_cache ? Hq + Hkv : Hq) * groups;
    const int v_items = write_cache ? Hkv * groups : 0;      // v: 8 values of each half per item
    const int idx = blockIdx.y * TW_ROPE_THREADS + threadIdx.x;
    if (idx >= rot_items + v_items) return;
    const bool is_v = idx >= rot_items;
    const int item = is_v ? idx - rot_items : idx;
    const int head = item / groups, i0 = (item - head * groups) * 8;
    const int col = (is_v ? (Hq + Hkv) * D : 0) + head * D + i0;
    uint4 lo = *reinterpret_cast<const uint4*>(row + col), hi = *reinterpret_cast<const uint4*>(row + col + half);
    __nv_bfloat162* lo2 = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* hi2 = reinterpret_cast<__nv_bfloat162*>(&hi);
    float blo[8], bhi[8];                       // col and half are multiples of 8: 32-byte aligned reads of the bias
    if (bias) {
        *reinterpret_cast<float4*>(blo) = *reinterpret_cast<const float4*>(bias + col);
        *reinterpret_cast<float4*>(blo + 4) = *reinterpret_cast<const float4*>(bias + col + 4);
        *reinterpret_cast<float4*>(bhi) = *reinterpret_cast<const float4*>(bias + col + half);
        *reinterpret_cast<float4*>(bhi + 4) = *reinterpret_cast<const float4*>(bias + col + half + 4);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float2 x1 = __bfloat1622float2(lo2[e]), x2 = __bfloat1622float2(hi2[e]);
        if (bias) {
            x1.x += blo[2 * e]; x1.y += blo[2 * e + 1];
            x2.x += bhi[2 * e]; x2.y += bhi[2 * e + 1];
        }
        float2 y1 = x1, y2 = x2;
        if (inv_freq && !is_v) {
            float sn = s_sin[i0 + 2 * e], cs = s_cos[i0 + 2 * e];
            y1.x = x1.x * cs - x2.x * sn; y2.x = x2.x * cs + x1.x * sn;
            sn = s_sin[i0 + 2 * e + 1]; cs = s_cos[i0 + 2 * e + 1];
            y1.y = x1.y * cs - x2.y * sn; y2.y = x2.y * cs + x1.y * sn;
        }
        lo2[e] = __floats2bfloat162_rn(y1.x, y1.y);
        hi2[e] = __floats2bfloat162_rn(y2.x, y2.y);
    }
    __nv_bfloat16* dst;
    if (!is_v && head < Hq) {
        dst = row + col;
    } else {
        if (page < 0) return;
        const int kvh = is_v ? head : head - Hq;
        dst = (is_v ? v_cache : k_cache) + (((size_t)page * Hkv + kvh) * page_size + in_page) * D + i0;
    }
    *reinterpret_cast<uint4*>(dst) = lo;
    *reinterpret_cast<uint4*>(dst + half) = hi;
}

TW_EXPORT int tw_rope_kv_write(void* qkv, int qkv_stride, const float* partial, int nsplit, long split_stride,
                               const float* bias, const int* positions,
                               const int* seq_of_token, const int* seq_slot, const int* block_table, int table_stride,
                               const float* inv_freq, void* k_cache, void* v_cache, int n_tokens, int Hq, int Hkv,
                               int D, int page_size, int num_pages, int write_cache, int dtype, int* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || (D & 1)) return (int)cudaErrorInvalidValue;
    if (dtype == TW_BF16 && !partial && (D & 15) == 0 && D <= 256 && (qkv_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(bias) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(qkv) & 15) == 0) {
        const int items = (Hq + 2 * Hkv) * (D / 16);
        const dim3 vgrid(n_tokens, (items + TW_ROPE_THREADS - 1) / TW_ROPE_THREADS);
        return tw_launch(rope_kv_write_bf16x8_kernel, vgrid, dim3(TW_ROPE_THREADS), 0, stream, 1, (__nv_bfloat16*)qkv,
                         qkv_stride, bias, positions, seq_of_token, seq_slot, block_table, table_stride, inv_freq,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, D, page_size, num_pages,
                         write_cache, status);
    }
    const int work = (Hq + 2 * Hkv) * (D / 2);
    const dim3 grid(n_tokens, (work + TW_ROPE_THREADS - 1) / TW_ROPE_THREADS);
    const int threads = TW_ROPE_THREADS;
    if (dtype == TW_F32)
        tw_launch(rope_kv_write_kernel<float>, dim3(grid), dim3(threads), 0, stream, 1, 
            (float*)qkv, qkv_stride, partial, nsplit, (size_t)split_stride, bias, positions, seq_of_token, seq_slot,
            block_table, table_stride, inv_freq,
            (float*)k_cache, (float*)v_cache, Hq, Hkv, D, page_size, num_pages, write_cache, status);
    else
        tw_launch(rope_kv_write_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, 1, 
            (__nv_bfloat16*)qkv, qkv_stride, partial, nsplit, (size_t)split_stride, bias, positions, seq_of_token,
            seq_slot, block_table, table_stride, inv_freq, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, D, page_size, num_pages, write_cache,
            status);
    return TW_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Rotation of pairs in place, on the first `n_heads` heads of each packed row and `rot_dims` values of a head
// from value `first` on: angle = float(position) * inv_freq[i]; pair i is (first + 2i, first + 2i+1) when
// `interleaved`, else (first + i, first + i + rot_dims / 2); cos and sin are both multiplied by `magnitude`.  The general form of the rotation above, for
// encodings no fused kernel takes.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rotate_pairs_kernel(T* __restrict__ rows, int row_stride, const int* __restrict__ positions,
                                    const int* __restrict__ seq_of_token, const float* __restrict__ inv_freq, int n_heads,
                                    int D, int first, int rot_dims, int interleaved, float magnitude) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    if (seq_of_token[n] < 0) return;
    const int pos = positions[n];
    const int half = rot_dims >> 1;
    T* row = rows + (size_t)n * row_stride;
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < n_heads * half; idx += gridDim.y * blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        const int a = head * D + first + (interleaved ? 2 * i : i), b = head * D + first + (interleaved ? 2 * i + 1 : i + half);
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        const float u = tw_to_float(row[a]), v = tw_to_float(row[b]);
        row[a] = tw_from_float<T>(u * cs - v * sn);
        row[b] = tw_from_float<T>(v * cs + u * sn);
    }
}

TW_EXPORT int tw_rotate_pairs(void* rows, int row_stride, const int* positions, const int* seq_of_token,
                              const float* inv_freq, int n_tokens, int n_heads, int D, int first, int rot_dims,
                              int interleaved, float magnitude, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || rot_dims < 2) return 0;
    if (first < 0 || first + rot_dims > D || (rot_dims & 1)) return (int)cudaErrorInvalidValue;
    const int work = n_heads * (rot_dims / 2);
    const dim3 grid(n_tokens, (work + 127) / 128 < 8 ? (work + 127) / 128 : 8);
    if (dtype == TW_F32)
        return tw_launch(rotate_pairs_kernel<float>, grid, dim3(128), 0, stream, 1, (float*)rows, row_stride, positions,
                         seq_of_token, inv_freq, n_heads, D, first, rot_dims, interleaved, magnitude);
    return tw_launch(rotate_pairs_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, (__nv_bfloat16*)rows, row_stride,
                     positions, seq_of_token, inv_freq, n_heads, D, first, rot_dims, interleaved, magnitude);
}

// ---------------------------------------------------------------------------
// RMS norm of spans of columns, in place: span s is `heads[s]` heads of `dim[s]` values from column `col[s]` on, and
// every head is normalised on its own, x <- x / sqrt(mean(x^2) + eps) * weight[s][i], with one weight [dim] for all
// heads of a span.  Statistics, quotient and product are fp32; one rounding to the rows' type.  Serves the
// per-head norms of queries and keys (two spans: the query heads, the key heads) and the norms of low-rank
// latents (a span of one head).  A warp per head.
// ---------------------------------------------------------------------------
struct NormSpans {
    int count;
    int col[2], heads[2], dim[2];
    const float* weight[2];
};

template <typename T>
__global__ void __launch_bounds__(128)
span_rmsnorm_kernel(T* __restrict__ rows, int row_stride, NormSpans sp, float eps, int n_rows, int heads_total) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= (long)n_rows * heads_total) return;
    const int row = (int)(item / heads_total);
    int head = (int)(item - (long)row * heads_total), s = 0;
    if (head >= sp.heads[0]) { head -= sp.heads[0]; s = 1; }
    const int D = sp.dim[s];
    T* x = rows + (size_t)row * row_stride + sp.col[s] + (size_t)head * D;
    const float* w = sp.weight[s];
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
        const float v = tw_to_float(x[i]);
        ss += v * v;
    }
    ss = tw_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    for (int i = lane; i < D; i += 32) x[i] = tw_from_float<T>((tw_to_float(x[i]) * inv) * w[i]);
}

TW_EXPORT int tw_span_rmsnorm(void* rows, int row_stride, int n_rows, int spans, int col0, int heads0, int dim0,
                              const float* weight0, int col1, int heads1, int dim1, const float* weight1, float eps,
                              int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (spans < 1 || spans > 2 || heads0 <= 0 || dim0 <= 0 || !weight0 || (spans == 2 && (heads1 <= 0 || dim1 <= 0 || !weight1)))
        return (int)cudaErrorInvalidValue;
    NormSpans sp;
    sp.count = spans;
    sp.col[0] = col0; sp.heads[0] = heads0; sp.dim[0] = dim0; sp.weight[0] = weight0;
    sp.col[1] = col1; sp.heads[1] = spans == 2 ? heads1 : 0; sp.dim[1] = dim1; sp.weight[1] = weight1;
    const int total = sp.heads[0] + sp.heads[1];
    const dim3 grid((unsigned)(((size_t)n_rows * total + 3) / 4));
    if (dtype == TW_F32)
        return tw_launch(span_rmsnorm_kernel<float>, grid, dim3(128), 0, stream, 1, (float*)rows, row_stride, sp, eps, n_rows, total);
    return tw_launch(span_rmsnorm_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, (__nv_bfloat16*)rows, row_stride, sp, eps,
                     n_rows, total);
}

// ---------------------------------------------------------------------------
// out[r, c] = x[r, c] * act(gate[r, c]) with act = sigmoid (1) or silu (2): an output gate on a mixer's heads.
// fp32 arithmetic, one rounding.  x, gate and out may be column slices of wider rows (strides in elements).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ x, int x_stride,
                                const T* __restrict__ gate, int gate_stride, int cols, long total, int act) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    for (; idx < total; idx += step) {
        const long r = idx / cols;
        const int c = (int)(idx - r * cols);
        const float g = tw_to_float(gate[r * gate_stride + c]);
        const float sg = 1.0f / (1.0f + expf(-g));
        out[r * out_stride + c] = tw_from_float<T>(tw_to_float(x[r * x_stride + c]) * (act == 2 ? g * sg : sg));
    }
}

TW_EXPORT int tw_gate_mul(void* out, int out_stride, const void* x, int x_stride, const void* gate, int gate_stride, int n_rows,
                          int cols, int act, int dtype, cudaStream_t stream) {
    if (n_rows <= 0 || cols <= 0) return 0;
    if (act != 1 && act != 2) return (int)cudaErrorInvalidValue;
    const long total = (long)n_rows * cols;
    const int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
    if (dtype == TW_F32)
        return tw_launch(gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, (float*)out, out_stride, (const float*)x,
                         x_stride, (const float*)gate, gate_stride, cols, total, act);
    return tw_launch(gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, (__nv_bfloat16*)out, out_stride,
                     (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)gate, gate_stride, cols, total, act);
}

// ---------------------------------------------------------------------------
// Soft cap of fp32 logits in place: x <- cap * tanh(x / cap).
// ---------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, long total, float cap) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    for (; idx < total; idx += step) x[idx] = cap * tanhf(x[idx] / cap);
}

TW_EXPORT int tw_softcap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    const int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
    return tw_launch(softcap_kernel, dim3(blocks), dim3(256), 0, stream, 1, x, (long)total, cap);
}

// ---------------------------------------------------------------------------
// SwiGLU activation: out[n, i] = silu(gate[n, i]) * up[n, i], silu(z) = z / (1 + exp(-z)),
// with gate = gate_up[n, i] and up = gate_up[n, I + i] (rows packed [gate; up]).
// Reference: flow_engine/model.py:76-80.
// ---------------------------------------------------------------------------
// With `interleaved` the columns come in groups of 16: eight gates, then their eight ups
// (the packing the fused small-batch kernel wants); otherwise all gates, then all ups.
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, long total,
                                int interleaved) {
    TW_TIMELINE_SCOPE(TW_K_SILU_MUL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    for (; idx < total; idx += step) {
        const long n = idx / inter;
        const int i = (int)(idx - n * inter);
        const int gcol = interleaved ? ((i >> 3) << 4) + (i & 7) : i;
        const int ucol = interleaved ? gcol + 8 : inter + i;
        const float g = tw_to_float(gate_up[n * 2 * inter + gcol]);
        const float u = tw_to_float(gate_up[n * 2 * inter + ucol]);
        const float act = g / (1.0f + expf(-g));
        out[idx] = tw_from_float<T>(act * u);
    }
}

// bf16 with the intermediate size a multiple of 8: a thread handles 8 outputs with 16-byte accesses.
__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate_up,
                                       int inter, long total8, int interleaved) {
    TW_TIMELINE_SCOPE(TW_K_SILU_MUL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    const int groups = inter >> 3;
    for (; idx < total8; idx += step) {
        const long n = idx / groups;
        const int j = (int)(idx - n * groups);
        const __nv_bfloat16* row = gate_up + n * 2 * (long)inter;
        const uint4 gv = *reinterpret_cast<const uint4*>(row + (interleaved ? j * 16 : j * 8));
        const uint4 uv = *reinterpret_cast<const uint4*>(row + (interleaved ? j * 16 + 8 : inter + j * 8));
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
            o2[e] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + n * (long)inter + j * 8) = ov;
    }
}

// The same from the fp32 slices of a gate/up product split over k ([slice][row][2 * inter], `split_stride` floats
// apart): the slices are added in the order every consumer of a split product uses (whole groups of four into
// four sums by slice mod 4, the rest into the first, then (s0 + s1) + (s2 + s3)), then silu(gate) * up, bf16 out.
// Four outputs per thread; inter a multiple of 8 when interleaved, of 4 otherwise.
__device__ __forceinline__ float4 tw_sum_slices4(const float* p, int nsplit, size_t split_stride) {
    float4 s[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    int k = 0;
    for (; k + 4 <= nsplit; k += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float4 v = *reinterpret_cast<const float4*>(p + (size_t)(k + u) * split_stride);
            s[u].x += v.x; s[u].y += v.y; s[u].z += v.z; s[u].w += v.w;
        }
    }
    for (; k < nsplit; ++k) {
        const float4 v = *reinterpret_cast<const float4*>(p + (size_t)k * split_stride);
        s[0].x += v.x; s[0].y += v.y; s[0].z += v.z; s[0].w += v.w;
    }
    return make_float4((s[0].x + s[1].x) + (s[2].x + s[3].x), (s[0].y + s[1].y) + (s[2].y + s[3].y),
                       (s[0].z + s[1].z) + (s[2].z + s[3].z), (s[0].w + s[1].w) + (s[2].w + s[3].w));
}

__global__ void silu_mul_slices_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ partial, int nsplit,
                                       size_t split_stride, int inter, long total4, int interleaved) {
    TW_TIMELINE_SCOPE(TW_K_SILU_MUL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    const int quads = inter >> 2;
    for (; idx < total4; idx += step) {
        const long n = idx / quads;
        const int i = (int)(idx - n * quads) * 4;                       // first of this thread's four outputs
        const int gcol = interleaved ? ((i >> 3) << 4) + (i & 7) : i;
        const int ucol = interleaved ? gcol + 8 : inter + i;
        const float* row = partial + (size_t)n * 2 * inter;
        const float4 g = tw_sum_slices4(row + gcol, nsplit, split_stride);
        const float4 u = tw_sum_slices4(row + ucol, nsplit, split_stride);
        uint2 packed;
        *reinterpret_cast<__nv_bfloat162*>(&packed.x) =
            __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        *reinterpret_cast<__nv_bfloat162*>(&packed.y) =
            __floats2bfloat162_rn(g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w);
        *reinterpret_cast<uint2*>(out + n * (long)inter + i) = packed;
    }
}

TW_EXPORT int tw_silu_mul_slices(void* out, const float* partial, int nsplit, long split_stride, int n_rows, int inter,
                                 int interleaved, cudaStream_t stream) {
    if (n_rows <= 0 || inter <= 0) return 0;
    if (nsplit < 1 || (inter & 3) || (interleaved && (inter & 7)) || (split_stride & 3) ||
        ((uintptr_t)partial & 15) || ((uintptr_t)out & 7))
        return (int)cudaErrorInvalidValue;
    const long total4 = (long)n_rows * (inter >> 2);
    const long blocks = (total4 + 255) / 256;
    tw_launch(silu_mul_slices_kernel, dim3((int)(blocks > 4096 ? 4096 : blocks)), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
              partial, nsplit, (size_t)split_stride, inter, total4, interleaved);
    return TW_LAUNCH_CHECK();
}

TW_EXPORT int tw_silu_mul(void* out, const void* gate_up, int n_rows, int inter, int interleaved, int dtype,
                          cudaStream_t stream) {
    const long total = (long)n_rows * inter;
    if (total <= 0) return 0;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    if (dtype == TW_BF16 && (inter & 7) == 0) {
        const long total8 = total >> 3;
        long b8 = (total8 + 255) / 256;
        if (b8 > 148L * 16) b8 = 148L * 16;
        tw_launch(silu_mul_bf16x8_kernel, dim3((int)b8), dim3(256), 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter,
                                                            total8, interleaved);
        return TW_LAUNCH_CHECK();
    }
    if (dtype == TW_F32)
        tw_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, 1, (float*)out, (const float*)gate_up, inter, total,
                                                                interleaved);
    else
        tw_launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                                                                        (const __nv_bfloat16*)gate_up, inter, total,
                                                                        interleaved);
    return TW_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// rows[n, c] += bias[c] over the first `cols` columns of each packed row, in place (fp32 sum, rounded once).
// For mixers whose bias is not added by the kernel that follows the projection.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_bias_rows_kernel(T* __restrict__ rows, int stride, const float* __restrict__ bias, int cols) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    T* row = rows + (size_t)blockIdx.x * stride;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) row[c] = tw_from_float<T>(tw_to_float(row[c]) + bias[c]);
}

TW_EXPORT int tw_add_bias_rows(void* rows, int stride, const float* bias, int n_rows, int cols, int dtype, cudaStream_t stream) {
    if (n_rows <= 0 || cols <= 0) return 0;
    if (dtype == TW_F32)
        return tw_launch(add_bias_rows_kernel<float>, dim3(n_rows), dim3(256), 0, stream, 1, (float*)rows, stride, bias, cols);
    return tw_launch(add_bias_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, 1, (__nv_bfloat16*)rows, stride,
                     bias, cols);
}

// ---------------------------------------------------------------------------
// Keys and values of the step's rows into their pages, as they stand in the packed rows (already biased and
// rotated): k [Hkv, Dk] at column k_col, v [Hkv, Dv] at column v_col; key rows and value rows of a page may
// differ in length.  Padding rows are skipped; a missing page sets the status bit.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ rows, int stride, int k_col, int v_col,
                                const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                const int* __restrict__ seq_slot, const int* __restrict__ block_table, int table_stride,
                                T* __restrict__ k_cache, T* __restrict__ v_cache, int Hkv, int Dk, int Dv, int page_size,
                                int num_pages, int* status) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;
    const int pos = positions[n];
    const int blk = pos / page_size, in_page = pos - blk * page_size;
    const int page = blk < table_stride ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, TW_ERR_PAGE);
        return;
    }
    const T* row = rows + (size_t)n * stride;
    for (int i = threadIdx.x; i < Hkv * Dk; i += blockDim.x) {
        const int h = i / Dk, d = i - h * Dk;
        k_cache[(((size_t)page * Hkv + h) * page_size + in_page) * Dk + d] = row[k_col + i];
    }
    if (!v_cache) return;        // the values are the keys: one set of pages
    for (int i = threadIdx.x; i < Hkv * Dv; i += blockDim.x) {
        const int h = i / Dv, d = i - h * Dv;
        v_cache[(((size_t)page * Hkv + h) * page_size + in_page) * Dv + d] = row[v_col + i];
    }
}

TW_EXPORT int tw_kv_store(const void* rows, int stride, int k_col, int v_col, const int* positions, const int* seq_of_token,
                          const int* seq_slot, const int* block_table, int table_stride, void* k_cache, void* v_cache,
                          int n_tokens, int Hkv, int Dk, int Dv, int page_size, int num_pages, int dtype, int* status,
                          cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dtype == TW_F32)
        return tw_launch(kv_store_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, 1, (const float*)rows, stride, k_col,
                         v_col, positions, seq_of_token, seq_slot, block_table, table_stride, (float*)k_cache, (float*)v_cache,
                         Hkv, Dk, Dv, page_size, num_pages, status);
    return tw_launch(kv_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, 1, (const __nv_bfloat16*)rows, stride,
                     k_col, v_col, positions, seq_of_token, seq_slot, block_table, table_stride, (__nv_bfloat16*)k_cache,
                     (__nv_bfloat16*)v_cache, Hkv, Dk, Dv, page_size, num_pages, status);
}

// ---------------------------------------------------------------------------
// What a token's projected row needs before an attention kernel can read the cache, in one pass (a block per token):
//   1. RMS norm of up to two spans of heads, as tw_span_rmsnorm does; span 0 may be written to rows of its own
//      (`dst0`, contiguous rows of heads0 * dim0 values) instead of in place;
//   2. rotation by position of `rot_dims` values from column `rot_col` on (one span that all heads share, outside
//      the normalised spans; pairs of neighbours or of halves), cos and sin multiplied by `magnitude`;
//   3. the store of the key columns (from `k_col`) and, where the values have pages of their own, of the value
//      columns (from `v_col`) into the token's place in its request's pages.
// Serves attention with normalised heads (spans: the query heads, the key heads; no rotation) and attention over
// low-rank latents (spans: the query latent, the key/value latent; the shared rotated key part; one set of pages).
// Everything between the loads and the stores is fp32; what is stored is what the rows hold afterwards, bit for bit.
// ---------------------------------------------------------------------------
#define TW_NRS_MAXV 8       // values of a head a thread keeps in registers in the block-wide form
template <typename T>
__global__ void __launch_bounds__(256)
norm_rotate_store_kernel(T* __restrict__ rows, int row_stride, NormSpans sp, T* __restrict__ dst0, float eps, int block_wide, int vec16,
                         int rot_col, int rot_dims, const float* __restrict__ inv_freq, int interleaved, float magnitude,
                         int k_col, int v_col, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                         const int* __restrict__ seq_slot, const int* __restrict__ block_table, int table_stride,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, int Hkv, int Dk, int Dv, int page_size, int num_pages,
                         int write_cache, int* status) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    T* row = rows + (size_t)n * row_stride;
    const int total = sp.heads[0] + sp.heads[1];
    // the token's place in the pages is looked up first: a chain of dependent loads that the norms then hide
    const int pos = positions[n];
    const int blk = pos / page_size, in_page = pos - blk * page_size;
    const int page = (write_cache && blk < table_stride) ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
    if (block_wide) {
        // few heads of many values (a latent): the whole block takes a head at a time, its values kept in registers
        __shared__ float scratch[33];
        for (int item = 0; item < total; ++item) {
            const int span = item < sp.heads[0] ? 0 : 1;
            const int head = span ? item - sp.heads[0] : item;
            const int D = sp.dim[span];
            T* x = row + sp.col[span] + (size_t)head * D;
            T* y = (span == 0 && dst0) ? dst0 + (size_t)n * sp.heads[0] * D + (size_t)head * D : x;
            const float* w = sp.weight[span];
            if constexpr (sizeof(T) == 2) {
                if (vec16) {
                    // rows, spans and weights on 16-byte boundaries: eight values per access, two accesses per thread
                    const int nv = D >> 3;
                    uint4 raw[2];
                    float ss8 = 0.f;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int i = threadIdx.x + j * blockDim.x;
                        raw[j] = make_uint4(0u, 0u, 0u, 0u);
                        if (i < nv) {
                            raw[j] = reinterpret_cast<const uint4*>(x)[i];
                            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 f = __bfloat1622float2(p2[e]);
                                ss8 += f.x * f.x + f.y * f.y;
                            }
                        }
                    }
                    ss8 = tw_block_sum(ss8, scratch);
                    const float inv8 = 1.0f / sqrtf(ss8 / (float)D + eps);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int i = threadIdx.x + j * blockDim.x;
                        if (i < nv) {
                            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
                            const float4 wa = reinterpret_cast<const float4*>(w)[2 * i], wb = reinterpret_cast<const float4*>(w)[2 * i + 1];
                            const float ww[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
                            uint4 packed;
                            __nv_bfloat162* q2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 f = __bfloat1622float2(p2[e]);
                                q2[e] = __floats2bfloat162_rn((f.x * inv8) * ww[2 * e], (f.y * inv8) * ww[2 * e + 1]);
                            }
                            reinterpret_cast<uint4*>(y)[i] = packed;
                        }
                    }
                    continue;
                }
            }
            float v[TW_NRS_MAXV];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < TW_NRS_MAXV; ++j) {
                const int i = threadIdx.x + j * blockDim.x;
                v[j] = i < D ? tw_to_float(x[i]) : 0.f;
                ss += v[j] * v[j];
            }
            for (int i = threadIdx.x + TW_NRS_MAXV * blockDim.x; i < D; i += blockDim.x) {      // heads wider than the registers hold
                const float u = tw_to_float(x[i]);
                ss += u * u;
            }
            ss = tw_block_sum(ss, scratch);
            const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
            for (int j = 0; j < TW_NRS_MAXV; ++j) {
                const int i = threadIdx.x + j * blockDim.x;
                if (i < D) y[i] = tw_from_float<T>((v[j] * inv) * w[i]);
            }
            for (int i = threadIdx.x + TW_NRS_MAXV * blockDim.x; i < D; i += blockDim.x)
                y[i] = tw_from_float<T>((tw_to_float(x[i]) * inv) * w[i]);
        }
    } else {
        for (int item = warp; item < total; item += warps) {
            const int span = item < sp.heads[0] ? 0 : 1;
            const int head = span ? item - sp.heads[0] : item;
            const int D = sp.dim[span];
            T* x = row + sp.col[span] + (size_t)head * D;
            T* y = (span == 0 && dst0) ? dst0 + (size_t)n * sp.heads[0] * D + (size_t)head * D : x;
            const float* w = sp.weight[span];
            float ss = 0.f;
            for (int i = lane; i < D; i += 32) {
                const float v = tw_to_float(x[i]);
                ss += v * v;
            }
            ss = tw_warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)D + eps);
            for (int i = lane; i < D; i += 32) y[i] = tw_from_float<T>((tw_to_float(x[i]) * inv) * w[i]);
        }
    }
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const int a = rot_col + (interleaved ? 2 * i : i), b = rot_col + (interleaved ? 2 * i + 1 : i + half);
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        const float u = tw_to_float(row[a]), v = tw_to_float(row[b]);
        row[a] = tw_from_float<T>(u * cs - v * sn);
        row[b] = tw_from_float<T>(v * cs + u * sn);
    }
    if (!write_cache) return;
    __syncthreads();            // the block's own writes to the row are visible to all of its threads from here on
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, TW_ERR_PAGE);
        return;
    }
    if constexpr (sizeof(T) == 2) {
        if (vec16) {            // (the launcher has checked that key and value rows start and end on 16-byte boundaries)
            const int kv8 = Dk >> 3;
            for (int i = threadIdx.x; i < Hkv * kv8; i += blockDim.x) {
                const int h = i / kv8, d = (i - h * kv8) << 3;
                *reinterpret_cast<uint4*>(k_cache + (((size_t)page * Hkv + h) * page_size + in_page) * Dk + d) =
                    *reinterpret_cast<const uint4*>(row + k_col + h * Dk + d);
            }
            if (!v_cache) return;
            const int vv8 = Dv >> 3;
            for (int i = threadIdx.x; i < Hkv * vv8; i += blockDim.x) {
                const int h = i / vv8, d = (i - h * vv8) << 3;
                *reinterpret_cast<uint4*>(v_cache + (((size_t)page * Hkv + h) * page_size + in_page) * Dv + d) =
                    *reinterpret_cast<const uint4*>(row + v_col + h * Dv + d);
            }
            return;
        }
    }
    for (int i = threadIdx.x; i < Hkv * Dk; i += blockDim.x) {
        const int h = i / Dk, d = i - h * Dk;
        k_cache[(((size_t)page * Hkv + h) * page_size + in_page) * Dk + d] = row[k_col + i];
    }
    if (!v_cache) return;        // the values are the keys: one set of pages
    for (int i = threadIdx.x; i < Hkv * Dv; i += blockDim.x) {
        const int h = i / Dv, d = i - h * Dv;
        v_cache[(((size_t)page * Hkv + h) * page_size + in_page) * Dv + d] = row[v_col + i];
    }
}

TW_EXPORT int tw_norm_rotate_store(void* rows, int row_stride, int n_tokens, int spans, int col0, int heads0, int dim0,
                                   const float* weight0, void* dst0, int col1, int heads1, int dim1, const float* weight1, float eps,
                                   int rot_col, int rot_dims, const float* inv_freq, int interleaved, float magnitude, int k_col,
                                   int v_col, const int* positions, const int* seq_of_token, const int* seq_slot,
                                   const int* block_table, int table_stride, void* k_cache, void* v_cache, int Hkv, int Dk, int Dv,
                                   int page_size, int num_pages, int write_cache, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (spans < 0 || spans > 2 || (spans >= 1 && (heads0 <= 0 || dim0 <= 0 || !weight0)) || (spans == 2 && (heads1 <= 0 || dim1 <= 0 || !weight1))
        || rot_dims < 0 || (rot_dims & 1) || (rot_dims && !inv_freq) || (write_cache && !k_cache))
        return (int)cudaErrorInvalidValue;
    NormSpans sp;
    sp.count = spans;
    sp.col[0] = col0; sp.heads[0] = spans >= 1 ? heads0 : 0; sp.dim[0] = dim0; sp.weight[0] = weight0;
    sp.col[1] = col1; sp.heads[1] = spans == 2 ? heads1 : 0; sp.dim[1] = dim1; sp.weight[1] = weight1;
    const int total = sp.heads[0] + sp.heads[1];
    // a warp per head where there are many heads; the whole block per head where there are few heads of many values
    const int widest = max(sp.heads[0] ? sp.dim[0] : 0, sp.heads[1] ? sp.dim[1] : 0);
    const int block_wide = (total > 0 && total <= 2 && widest >= 128) ? 1 : 0;
    const int threads = (block_wide ? widest >= 1024 : total >= 8) ? 256 : 128;
    // 16-byte accesses (bfloat16 only): every span, the key and value columns, the rows and the pages start and end on
    // 16-byte boundaries, and a head fits two accesses per thread
    auto a16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    int vec16 = (dtype != TW_F32 && a16(rows) && a16(dst0) && a16(k_cache) && a16(v_cache) && a16(weight0) && a16(weight1)
                 && (row_stride & 7) == 0 && (k_col & 7) == 0 && (Dk & 7) == 0 && (!v_cache || ((v_col & 7) == 0 && (Dv & 7) == 0))) ? 1 : 0;
    for (int sidx = 0; sidx < 2; ++sidx)
        if (sp.heads[sidx] && ((sp.col[sidx] & 7) || (sp.dim[sidx] & 7) || (block_wide && sp.dim[sidx] > 16 * threads))) vec16 = 0;
    if (dtype == TW_F32)
        return tw_launch(norm_rotate_store_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, 1, (float*)rows, row_stride, sp,
                         (float*)dst0, eps, block_wide, 0, rot_col, rot_dims, inv_freq, interleaved, magnitude, k_col, v_col, positions, seq_of_token,
                         seq_slot, block_table, table_stride, (float*)k_cache, (float*)v_cache, Hkv, Dk, Dv, page_size, num_pages,
                         write_cache, status);
    return tw_launch(norm_rotate_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, 1, (__nv_bfloat16*)rows,
                     row_stride, sp, (__nv_bfloat16*)dst0, eps, block_wide, vec16, rot_col, rot_dims, inv_freq, interleaved, magnitude, k_col, v_col,
                     positions, seq_of_token, seq_slot, block_table, table_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                     Hkv, Dk, Dv, page_size, num_pages, write_cache, status);
}

// ---------------------------------------------------------------------------
// acc = (first ? 0 : acc) + scale * x, element by element in fp32; `out` (may be null) receives the new acc in
// the activation type.  For mixers whose result is a weighted sum of several mixers' results.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void scaled_accumulate_kernel(float* __restrict__ acc, T* __restrict__ out, const T* __restrict__ x, float scale,
                                         int first, size_t count) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float v = (first ? 0.f : acc[i]) + scale * tw_to_float(x[i]);
    acc[i] = v;
    if (out) out[i] = tw_from_float<T>(v);
}

TW_EXPORT int tw_scaled_accumulate(float* acc, void* out, const void* x, float scale, int first, long long count, int dtype,
                                   cudaStream_t stream) {
    if (count <= 0) return 0;
    const dim3 grid((unsigned)((count + 255) / 256));
    if (dtype == TW_F32)
        return tw_launch(scaled_accumulate_kernel<float>, grid, dim3(256), 0, stream, 1, acc, (float*)out, (const float*)x, scale,
                         first, (size_t)count);
    return tw_launch(scaled_accumulate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 1, acc, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)x, scale, first, (size_t)count);
}

// ---------------------------------------------------------------------------
// out[n] = sum_m scale_m * x_m[n] (weights null), or sum_m scale_m * x_m[n] / sqrt(mean(x_m[n]^2) + eps) * weight_m, for up
// to TW_SUM_MEMBERS members whose rows lie in buffers of their own: one pass, statistics and sum in fp32 (the members
// are added in their order), one rounding.  A row is read twice, the second time from cache.
// ---------------------------------------------------------------------------
#define TW_SUM_MEMBERS 4
struct SumMembers {
    const void* x[TW_SUM_MEMBERS];
    float scale[TW_SUM_MEMBERS];
};

template <typename T>
__global__ void __launch_bounds__(TW_NORM_THREADS)
weighted_sum_rows_kernel(T* __restrict__ out, const SumMembers in, const float* __restrict__ weights, float eps, int members,
                         int width) {
    __shared__ float scratch[33];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const size_t base = (size_t)blockIdx.x * width;
    float f[TW_SUM_MEMBERS];
#pragma unroll
    for (int m = 0; m < TW_SUM_MEMBERS; ++m) {
        f[m] = in.scale[m];
        if (m < members && weights) {        // (the same for every thread of the block)
            const T* x = (const T*)in.x[m] + base;
            float ss = 0.f;
            for (int c = threadIdx.x; c < width; c += blockDim.x) {
                const float v = tw_to_float(x[c]);
                ss += v * v;
            }
            ss = tw_block_sum(ss, scratch);
            f[m] = in.scale[m] / sqrtf(ss / (float)width + eps);
        }
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < TW_SUM_MEMBERS; ++m) {
            if (m < members) {
                const float v = tw_to_float(((const T*)in.x[m])[base + c]);
                acc += weights ? v * f[m] * weights[(size_t)m * width + c] : f[m] * v;
            }
        }
        out[base + c] = tw_from_float<T>(acc);
    }
}

TW_EXPORT int tw_weighted_sum_rows(void* out, const void* x0, const void* x1, const void* x2, const void* x3, float s0, float s1,
                                   float s2, float s3, const float* weights, float eps, int members, int n_rows, int width,
                                   int dtype, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    if (members < 1 || members > TW_SUM_MEMBERS) return (int)cudaErrorInvalidValue;
    SumMembers in;
    in.x[0] = x0; in.x[1] = x1; in.x[2] = x2; in.x[3] = x3;
    in.scale[0] = s0; in.scale[1] = s1; in.scale[2] = s2; in.scale[3] = s3;
    if (dtype == TW_F32)
        return tw_launch(weighted_sum_rows_kernel<float>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, (float*)out, in,
                         weights, eps, members, width);
    return tw_launch(weighted_sum_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1,
                     (__nv_bfloat16*)out, in, weights, eps, members, width);
}

// ---------------------------------------------------------------------------
// resid[n, :] += vec for the first n_rows rows: a learned vector added to every row of the fp32 residual stream.
// ---------------------------------------------------------------------------
__global__ void add_row_vector_kernel(float* __restrict__ resid, const float* __restrict__ vec, int width, size_t count) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) resid[i] += vec[i % width];
}

TW_EXPORT int tw_add_row_vector(float* resid, const float* vec, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    const size_t count = (size_t)n_rows * width;
    return tw_launch(add_row_vector_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, 1, resid, vec, width, count);
}

// ---------------------------------------------------------------------------
// resid += delta in fp32, where delta is a tensor of the activation type or the fp32 slices of a split product
// (added in slice order first).  For blocks that add a sub-layer's result without a norm behind it.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_delta_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ partial,
                                 int nsplit, size_t split_stride, size_t count) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float d = 0.f;
    if (partial) {
        for (int k = 0; k < nsplit; ++k) d += partial[(size_t)k * split_stride + i];
    } else {
        d = tw_to_float(delta[i]);
    }
    resid[i] += d;
}

TW_EXPORT int tw_add_delta(float* resid, const void* delta, const float* partial, int nsplit, long long split_stride,
                           long long count, int dtype, cudaStream_t stream) {
    if (count <= 0) return 0;
    const dim3 grid((unsigned)((count + 255) / 256));
    if (dtype == TW_F32)
        return tw_launch(add_delta_kernel<float>, grid, dim3(256), 0, stream, 1, resid, (const float*)delta, partial, nsplit,
                         (size_t)split_stride, (size_t)count);
    return tw_launch(add_delta_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 1, resid, (const __nv_bfloat16*)delta, partial,
                     nsplit, (size_t)split_stride, (size_t)count);
}

// ---------------------------------------------------------------------------
// acc[n] = (first ? 0 : acc[n]) + scale * x[n] / sqrt(mean(x[n]^2) + eps) * weight, row by row in fp32; `out` (may be
// null) receives the new acc in the activation type.  For mixers that normalise each member's result before the sum.
// ---------------------------------------------------------------------------
template <typename T, bool ONE_PASS>
__global__ void __launch_bounds__(TW_NORM_THREADS)
normed_accumulate_kernel(float* __restrict__ acc, T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ weight,
                         float eps, float scale, int first, int width) {
    __shared__ float scratch[33];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const size_t base = (size_t)blockIdx.x * width;
    if (ONE_PASS) {
        // the row, the old sum and the weight are all asked for before the first of them is needed
        float v[TW_NORM_MAXV], a[TW_NORM_MAXV], wt[TW_NORM_MAXV];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int c = threadIdx.x + j * TW_NORM_THREADS;
            const bool in = c < width;
            v[j] = in ? tw_to_float(x[base + c]) : 0.f;
            a[j] = (in && !first) ? acc[base + c] : 0.f;
            wt[j] = in ? weight[c] : 0.f;
            ss += v[j] * v[j];
        }
        ss = tw_block_sum(ss, scratch);
        const float f = scale / sqrtf(ss / (float)width + eps);
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int c = threadIdx.x + j * TW_NORM_THREADS;
            if (c < width) {
                const float r = a[j] + v[j] * f * wt[j];
                acc[base + c] = r;
                if (out) out[base + c] = tw_from_float<T>(r);
            }
        }
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = tw_to_float(x[base + c]);
        ss += v * v;
    }
    ss = tw_block_sum(ss, scratch);
    const float f = scale / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = (first ? 0.f : acc[base + c]) + tw_to_float(x[base + c]) * f * weight[c];
        acc[base + c] = v;
        if (out) out[base + c] = tw_from_float<T>(v);
    }
}

TW_EXPORT int tw_normed_accumulate(float* acc, void* out, const void* x, const float* weight, float eps, float scale, int first,
                                   int n_rows, int width, int dtype, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    const bool one = width <= TW_NORM_THREADS * TW_NORM_MAXV;
    if (dtype == TW_F32)
        return tw_launch(one ? normed_accumulate_kernel<float, true> : normed_accumulate_kernel<float, false>, dim3(n_rows),
                         dim3(TW_NORM_THREADS), 0, stream, 1, acc, (float*)out, (const float*)x, weight, eps, scale, first, width);
    return tw_launch(one ? normed_accumulate_kernel<__nv_bfloat16, true> : normed_accumulate_kernel<__nv_bfloat16, false>,
                     dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, acc, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, weight,
                     eps, scale, first, width);
}
