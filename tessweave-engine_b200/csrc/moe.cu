// Routed feed-forward (mixture of experts), weight-streaming form: every (token, chosen expert) pair is a
// matrix-vector product of its own.  Steps with few tokens are bound by the bytes of the chosen experts'
// matrices, which these kernels stream once per pair in 16-byte loads.
//
//   tw_moe_route     z = Wr h + br (fp32); the `top` largest z (lowest index first at a tie); their weights are the
//                    softmax over those alone; optionally one more dot product per token, sigmoid(ws . h), the
//                    gate of an expert that every token uses.  With `scoring` 1: s = softmax(z) over every router
//                    output, the `top` largest s + correction are chosen, and their weights are s * weight_scale
//                    (not renormalised)
//   tw_moe_gate_up   act[token, j] = silu(Wg_e h) * (Wu_e h)          e = the j-th expert of the token
//                    with `act` 1: g = min(Wg_e h, limit), u = clamp(Wu_e h, -limit, limit), g sigmoid(alpha g) (u + 1)
//   tw_moe_down      out[token] = sum_j weight_j Wd_e act[token, j]  (+ gate * shared[token])
//
// The router may have more outputs than there are experts with matrices: outputs E .. E + identity - 1 are identity
// experts, whose output is the token's row itself (times the weight); they read no matrix.
//
// Expert matrices are stacked: gate/up [E, 2, F, width] (a gate matrix followed by its up matrix), down
// [E, width, F].  Dot products accumulate in fp32; the weighted sum over experts is fp32.
#include "common.cuh"

template <typename T>
__device__ __forceinline__ float tw_dot_row(const T* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.f;
    for (int i = lane; i < n; i += 32) acc += tw_to_float(w[i]) * x[i];
    return tw_warp_sum(acc);
}

// bf16 rows whose length is a multiple of 8 and whose start is 16-byte aligned: eight values per load, four
// loads of a lane under way at a time (a row is streamed once; what bounds it is how much is in flight)
__device__ __forceinline__ float tw_fma8(uint4 raw, const float* __restrict__ x, float acc) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        acc += f.x * x[2 * e] + f.y * x[2 * e + 1];
    }
    return acc;
}

__device__ __forceinline__ uint4 tw_stream16(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float tw_dot_row8(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int i = lane * 8;
    for (; i + 768 < n; i += 1024) {
        const uint4 r0 = tw_stream16(w + i), r1 = tw_stream16(w + i + 256), r2 = tw_stream16(w + i + 512), r3 = tw_stream16(w + i + 768);
        a0 = tw_fma8(r0, x + i, a0); a1 = tw_fma8(r1, x + i + 256, a1);
        a2 = tw_fma8(r2, x + i + 512, a2); a3 = tw_fma8(r3, x + i + 768, a3);
    }
    for (; i < n; i += 256) a0 = tw_fma8(tw_stream16(w + i), x + i, a0);
    return tw_warp_sum((a0 + a1) + (a2 + a3));
}

// two rows of equal length at once (an expert's gate row and its up row): eight loads of a lane under way
__device__ __forceinline__ void tw_dot2_row8(const __nv_bfloat16* __restrict__ wa, const __nv_bfloat16* __restrict__ wb,
                                             const float* __restrict__ x, const float* __restrict__ y, int n, int lane,
                                             float& da, float& db) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
    int i = lane * 8;
    for (; i + 768 < n; i += 1024) {
        const uint4 r0 = tw_stream16(wa + i), r1 = tw_stream16(wa + i + 256), r2 = tw_stream16(wa + i + 512), r3 = tw_stream16(wa + i + 768);
        const uint4 s0 = tw_stream16(wb + i), s1 = tw_stream16(wb + i + 256), s2 = tw_stream16(wb + i + 512), s3 = tw_stream16(wb + i + 768);
        a0 = tw_fma8(r0, x + i, a0); a1 = tw_fma8(r1, x + i + 256, a1); a2 = tw_fma8(r2, x + i + 512, a2); a3 = tw_fma8(r3, x + i + 768, a3);
        b0 = tw_fma8(s0, y + i, b0); b1 = tw_fma8(s1, y + i + 256, b1); b2 = tw_fma8(s2, y + i + 512, b2); b3 = tw_fma8(s3, y + i + 768, b3);
    }
    for (; i < n; i += 256) {
        a0 = tw_fma8(tw_stream16(wa + i), x + i, a0);
        b0 = tw_fma8(tw_stream16(wb + i), y + i, b0);
    }
    da = tw_warp_sum((a0 + a1) + (a2 + a3));
    db = tw_warp_sum((b0 + b1) + (b2 + b3));
}

template <typename T> __device__ __forceinline__ float tw_dot(const T* w, const float* x, int n, int lane, bool vec);
template <> __device__ __forceinline__ float tw_dot<float>(const float* w, const float* x, int n, int lane, bool) {
    return tw_dot_row(w, x, n, lane);
}
template <> __device__ __forceinline__ float tw_dot<__nv_bfloat16>(const __nv_bfloat16* w, const float* x, int n, int lane, bool vec) {
    return vec ? tw_dot_row8(w, x, n, lane) : tw_dot_row(w, x, n, lane);
}

// da = wa . x and db = wb . y, the two rows streamed side by side
template <typename T> __device__ __forceinline__ void tw_dot2(const T* wa, const T* wb, const float* x, const float* y, int n, int lane,
                                                              bool vec, float& da, float& db);
template <> __device__ __forceinline__ void tw_dot2<float>(const float* wa, const float* wb, const float* x, const float* y, int n,
                                                           int lane, bool, float& da, float& db) {
    da = tw_dot_row(wa, x, n, lane);
    db = tw_dot_row(wb, y, n, lane);
}
template <> __device__ __forceinline__ void tw_dot2<__nv_bfloat16>(const __nv_bfloat16* wa, const __nv_bfloat16* wb, const float* x,
                                                                   const float* y, int n, int lane, bool vec, float& da, float& db) {
    if (vec) { tw_dot2_row8(wa, wb, x, y, n, lane, da, db); return; }
    da = tw_dot_row(wa, x, n, lane);
    db = tw_dot_row(wb, y, n, lane);
}

template <typename T>
__global__ void __launch_bounds__(512)
moe_route_kernel(int* __restrict__ chosen, float* __restrict__ weight, float* __restrict__ shared_gate,
                 const T* __restrict__ h, int h_stride, const T* __restrict__ wr, const float* __restrict__ br,
                 const T* __restrict__ ws, int width, int E, int top, int scoring, const float* __restrict__ correction,
                 float weight_scale) {
    extern __shared__ float sm[];           // [width] the row, [E + 1] logits, [E] marks
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* x = sm;
    float* z = sm + width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) x[c] = tw_to_float(h[(size_t)row * h_stride + c]);
    __syncthreads();
    const bool vec = (width & 7) == 0;
    for (int e = warp; e < E + (ws ? 1 : 0); e += (int)(blockDim.x >> 5)) {
        const float d = tw_dot<T>(e < E ? wr + (size_t)e * width : ws, x, width, lane, vec);
        if (lane == 0) z[e] = e < E ? d + (br ? br[e] : 0.f) : d;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    if (ws && shared_gate) shared_gate[row] = 1.0f / (1.0f + expf(-z[E]));
    // selection: `top` times the largest logit that is left; a row of NaN still names `top` different experts
    float* taken = z + E + 1;
    for (int e = 0; e < E; ++e) taken[e] = 0.f;
    if (scoring == 1) {
        // scores over every output; the choice looks at score + correction, the weight is the plain score
        float top_z = -INFINITY, den = 0.f;
        for (int e = 0; e < E; ++e) top_z = fmaxf(top_z, z[e]);
        for (int e = 0; e < E; ++e) { z[e] = expf(z[e] - top_z); den += z[e]; }
        for (int e = 0; e < E; ++e) z[e] /= den;
        for (int j = 0; j < top; ++j) {
            int arg = -1;
            float best = -INFINITY;
            for (int e = 0; e < E; ++e) {
                if (taken[e] != 0.f) continue;
                const float c = z[e] + (correction ? correction[e] : 0.f);
                if (arg < 0 || c > best) { arg = e; best = c; }
            }
            taken[arg] = 1.f;
            chosen[(size_t)row * top + j] = arg;
            weight[(size_t)row * top + j] = z[arg] * weight_scale;
        }
        return;
    }
    float best0 = 0.f, sum = 0.f;
    for (int j = 0; j < top; ++j) {
        int arg = -1;
        float best = -INFINITY;
        for (int e = 0; e < E; ++e) {
            if (taken[e] != 0.f) continue;
            if (arg < 0 || z[e] > best) { arg = e; best = z[e]; }
        }
        taken[arg] = 1.f;
        chosen[(size_t)row * top + j] = arg;
        if (j == 0) best0 = best;
        const float w = expf(best - best0);
        weight[(size_t)row * top + j] = w;
        sum += w;
    }
    for (int j = 0; j < top; ++j) weight[(size_t)row * top + j] /= sum;
}

TW_EXPORT int tw_moe_route(int* chosen, float* weight, float* shared_gate, const void* h, int h_stride, const void* wr,
                           const float* br, const void* ws, int rows, int width, int E, int top, int scoring,
                           const float* correction, float weight_scale, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || scoring < 0 || scoring > 1) return (int)cudaErrorInvalidValue;
    const size_t smem = ((size_t)width + 2 * E + 1) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const int threads = 32 * min(16, max(4, E + 1));        // a warp per expert (and one for the shared gate), up to 16
    if (dtype == TW_F32)
        return tw_launch(moe_route_kernel<float>, dim3(rows), dim3(threads), smem, stream, 1, chosen, weight, shared_gate,
                         (const float*)h, h_stride, (const float*)wr, br, (const float*)ws, width, E, top, scoring, correction,
                         weight_scale);
    return tw_launch(moe_route_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), smem, stream, 1, chosen, weight, shared_gate,
                     (const __nv_bfloat16*)h, h_stride, (const __nv_bfloat16*)wr, br, (const __nv_bfloat16*)ws, width, E, top,
                     scoring, correction, weight_scale);
}

#define TW_MOE_WARPS 8

// what an expert makes of its gate and up products: 0 silu(g) u;  1 with g = min(g, limit), u = clamp(u, -limit, limit):
// g sigmoid(alpha g) (u + 1)
__device__ __forceinline__ float tw_glu(float g, float u, int act, float limit, float alpha) {
    if (act == 1) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    }
    return g / (1.0f + expf(-g)) * u;
}

template <typename T>
__global__ void __launch_bounds__(32 * TW_MOE_WARPS)
moe_gate_up_kernel(T* __restrict__ act, const T* __restrict__ h, int h_stride, const T* __restrict__ wgu,
                   const int* __restrict__ chosen, int width, int F, int E, int top, int rows_per_block, int glu, float limit,
                   float alpha) {
    extern __shared__ float sm[];           // [width]
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int pair = blockIdx.x, row = pair / top;
    const int e = chosen[pair];
    if (e < 0 || e >= E) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int c = threadIdx.x; c < width; c += blockDim.x) sm[c] = tw_to_float(h[(size_t)row * h_stride + c]);
    __syncthreads();
    const bool vec = (width & 7) == 0;
    const T* wg = wgu + (size_t)e * 2 * F * width;
    const T* wu = wg + (size_t)F * width;
    const int f0 = blockIdx.y * rows_per_block, f1 = min(F, f0 + rows_per_block);
    for (int f = f0 + warp; f < f1; f += TW_MOE_WARPS) {
        float g, u;
        tw_dot2<T>(wg + (size_t)f * width, wu + (size_t)f * width, sm, sm, width, lane, vec, g, u);
        if (lane == 0) act[(size_t)pair * F + f] = tw_from_float<T>(tw_glu(g, u, glu, limit, alpha));
    }
}

TW_EXPORT int tw_moe_gate_up(void* act, const void* h, int h_stride, const void* wgu, const int* chosen, int rows, int width,
                             int F, int E, int top, int glu, float limit, float alpha, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    // enough blocks to fill the GPU when there are few pairs, whole rounds of warps per block
    int per = F;
    while (per > 4 * TW_MOE_WARPS && (size_t)rows * top * ((F + per - 1) / per) < 592) per = (per + 1) / 2;
    per = ((per + TW_MOE_WARPS - 1) / TW_MOE_WARPS) * TW_MOE_WARPS;
    const dim3 grid(rows * top, (F + per - 1) / per);
    if (dtype == TW_F32)
        return tw_launch(moe_gate_up_kernel<float>, grid, dim3(32 * TW_MOE_WARPS), smem, stream, 1, (float*)act, (const float*)h,
                         h_stride, (const float*)wgu, chosen, width, F, E, top, per, glu, limit, alpha);
    return tw_launch(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(32 * TW_MOE_WARPS), smem, stream, 1, (__nv_bfloat16*)act,
                     (const __nv_bfloat16*)h, h_stride, (const __nv_bfloat16*)wgu, chosen, width, F, E, top, per, glu, limit, alpha);
}

template <typename T>
__global__ void __launch_bounds__(32 * TW_MOE_WARPS)
moe_down_kernel(T* __restrict__ out, const T* __restrict__ act, const T* __restrict__ wd, const int* __restrict__ chosen,
                const float* __restrict__ weight, const T* __restrict__ shared, const float* __restrict__ shared_gate,
                int width, int F, int E, int top, int cols_per_block, const T* __restrict__ h, int h_stride, int identity) {
    extern __shared__ float sm[];           // [top][F] the activations of the token's experts
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < top * F; i += blockDim.x) sm[i] = tw_to_float(act[(size_t)row * top * F + i]);
    __syncthreads();
    const bool vec = (F & 7) == 0;
    const float sg = shared ? (shared_gate ? shared_gate[row] : 1.f) : 0.f;
    const int c0 = blockIdx.y * cols_per_block, c1 = min(width, c0 + cols_per_block);
    for (int c = c0 + warp; c < c1; c += TW_MOE_WARPS) {
        float acc = 0.f;
        int j = 0;
        for (; j + 1 < top; j += 2) {            // two experts' rows side by side; always added in the order of the experts
            const int e0 = chosen[(size_t)row * top + j], e1 = chosen[(size_t)row * top + j + 1];
            if (e0 < 0 || e0 >= E || e1 < 0 || e1 >= E) {
                if (identity > 0) {          // one of the two has no matrices: each on its own
                    for (int jj = j; jj < j + 2; ++jj) {
                        const int e = chosen[(size_t)row * top + jj];
                        if (e >= E && e < E + identity)
                            acc += weight[(size_t)row * top + jj] * tw_to_float(h[(size_t)row * h_stride + c]);
                        else if (e >= 0 && e < E)
                            acc += weight[(size_t)row * top + jj] * tw_dot<T>(wd + ((size_t)e * width + c) * F, sm + (size_t)jj * F, F, lane, vec);
                    }
                }
                continue;
            }
            float d0, d1;
            tw_dot2<T>(wd + ((size_t)e0 * width + c) * F, wd + ((size_t)e1 * width + c) * F, sm + (size_t)j * F, sm + (size_t)(j + 1) * F,
                       F, lane, vec, d0, d1);
            acc += weight[(size_t)row * top + j] * d0;
            acc += weight[(size_t)row * top + j + 1] * d1;
        }
        for (; j < top; ++j) {
            const int e = chosen[(size_t)row * top + j];
            if (e >= E && e < E + identity) acc += weight[(size_t)row * top + j] * tw_to_float(h[(size_t)row * h_stride + c]);
            if (e < 0 || e >= E) continue;
            acc += weight[(size_t)row * top + j] * tw_dot<T>(wd + ((size_t)e * width + c) * F, sm + (size_t)j * F, F, lane, vec);
        }
        if (lane == 0) {
            if (shared) acc += sg * tw_to_float(shared[(size_t)row * width + c]);
            out[(size_t)row * width + c] = tw_from_float<T>(acc);
        }
    }
}

TW_EXPORT int tw_moe_down(void* out, const void* act, const void* wd, const int* chosen, const float* weight,
                          const void* shared, const float* shared_gate, int rows, int width, int F, int E, int top,
                          const void* h, int h_stride, int identity, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (identity < 0 || (identity > 0 && !h)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)top * F * sizeof(float);
    if (smem > 160 * 1024) return (int)cudaErrorInvalidValue;
    int per = width;
    while (per > TW_MOE_WARPS && (size_t)rows * ((width + per - 1) / per) < 592) per = (per + 1) / 2;
    per = ((per + TW_MOE_WARPS - 1) / TW_MOE_WARPS) * TW_MOE_WARPS;
    const dim3 grid(rows, (width + per - 1) / per);
    if (dtype == TW_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tw_launch(moe_down_kernel<float>, grid, dim3(32 * TW_MOE_WARPS), smem, stream, 1, (float*)out, (const float*)act,
                         (const float*)wd, chosen, weight, (const float*)shared, shared_gate, width, F, E, top, per,
                         (const float*)h, h_stride, identity);
    }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(moe_down_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return tw_launch(moe_down_kernel<__nv_bfloat16>, grid, dim3(32 * TW_MOE_WARPS), smem, stream, 1, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)act, (const __nv_bfloat16*)wd, chosen, weight, (const __nv_bfloat16*)shared,
                     shared_gate, width, F, E, top, per, (const __nv_bfloat16*)h, h_stride, identity);
}

// ---------------------------------------------------------------------------
// Steps with many rows: the (token, expert) pairs are sorted by expert, so that each expert's rows stand together
// and its matrices meet them in one product with many rows.
//
//   tw_moe_sort      order[i] = the pair (token * top + j) at sorted place i (-1 behind the last group); place[pair] = its place;
//                    ends[e] = one past the last place of expert e (the prefix sum of the experts' counts)
//   tw_moe_gather    xs[i] = h[order[i] / top]
//   tw_moe_combine   out[token] = sum_j weight[token, j] * ys[place[token * top + j]]  (+ gate * shared[token]);
//                    a pair whose expert is an identity expert has no place and adds weight * h[token]
//   tw_glu_rows      act = what an expert makes of its gate and up products, over rows [gates | ups]
//
// The order of the pairs inside an expert's group is whatever the atomics give; no result depends on it.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_sort_kernel(int* __restrict__ order, int* __restrict__ place, int* __restrict__ ends, const int* __restrict__ chosen,
                int pairs, int E) {
    extern __shared__ int cnt[];            // [E] counts, then [E] running starts
    tw_grid_wait();
    tw_grid_launch_dependents();
    int* start = cnt + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = run;
            run += cnt[e];
            ends[e] = run;
        }
    }
    __syncthreads();
    // places behind the last group (pairs whose expert has no matrices) name no pair
    for (int p = ends[E - 1] + threadIdx.x; p < pairs; p += blockDim.x) order[p] = -1;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < E) {
            const int at = atomicAdd(&start[e], 1);
            order[at] = p;
            place[p] = at;
        } else {
            place[p] = -1;
        }
    }
}

TW_EXPORT int tw_moe_sort(int* order, int* place, int* ends, const int* chosen, int pairs, int E, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (E <= 0 || E > 4096) return (int)cudaErrorInvalidValue;
    return tw_launch(moe_sort_kernel, dim3(1), dim3(1024), 2 * (size_t)E * sizeof(int), stream, 1, order, place, ends, chosen,
                     pairs, E);
}

template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ xs, const T* __restrict__ h, int h_stride, const int* __restrict__ order,
                                  int top, int width) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int i = blockIdx.x;
    if (order[i] < 0) {         // a place no pair was sorted into: a row of zeros, which no group's product reads
        for (int c = threadIdx.x; c < width; c += blockDim.x) xs[(size_t)i * width + c] = tw_from_float<T>(0.f);
        return;
    }
    const T* src = h + (size_t)(order[i] / top) * h_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[(size_t)i * width + c] = src[c];
}

TW_EXPORT int tw_moe_gather(void* xs, const void* h, int h_stride, const int* order, int pairs, int top, int width, int dtype,
                            cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (dtype == TW_F32)
        return tw_launch(moe_gather_kernel<float>, dim3(pairs), dim3(256), 0, stream, 1, (float*)xs, (const float*)h, h_stride,
                         order, top, width);
    return tw_launch(moe_gather_kernel<__nv_bfloat16>, dim3(pairs), dim3(256), 0, stream, 1, (__nv_bfloat16*)xs,
                     (const __nv_bfloat16*)h, h_stride, order, top, width);
}

template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ ys, const int* __restrict__ place,
                                   const float* __restrict__ weight, const T* __restrict__ shared,
                                   const float* __restrict__ shared_gate, int top, int width, const int* __restrict__ chosen,
                                   const T* __restrict__ h, int h_stride, int E, int identity) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row = blockIdx.x;
    const float sg = shared ? (shared_gate ? shared_gate[row] : 1.f) : 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const int at = place[(size_t)row * top + j];
            if (at >= 0) acc += weight[(size_t)row * top + j] * tw_to_float(ys[(size_t)at * width + c]);
            else if (identity > 0) {
                const int e = chosen[(size_t)row * top + j];
                if (e >= E && e < E + identity) acc += weight[(size_t)row * top + j] * tw_to_float(h[(size_t)row * h_stride + c]);
            }
        }
        if (shared) acc += sg * tw_to_float(shared[(size_t)row * width + c]);
        out[(size_t)row * width + c] = tw_from_float<T>(acc);
    }
}

TW_EXPORT int tw_moe_combine(void* out, const void* ys, const int* place, const float* weight, const void* shared,
                             const float* shared_gate, int rows, int top, int width, const int* chosen, const void* h,
                             int h_stride, int E, int identity, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (identity < 0 || (identity > 0 && (!h || !chosen))) return (int)cudaErrorInvalidValue;
    if (dtype == TW_F32)
        return tw_launch(moe_combine_kernel<float>, dim3(rows), dim3(256), 0, stream, 1, (float*)out, (const float*)ys, place,
                         weight, (const float*)shared, shared_gate, top, width, chosen, (const float*)h, h_stride, E, identity);
    return tw_launch(moe_combine_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)ys, place, weight, (const __nv_bfloat16*)shared, shared_gate, top, width, chosen,
                     (const __nv_bfloat16*)h, h_stride, E, identity);
}

template <typename T>
__global__ void glu_rows_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, long total, int glu, float limit,
                                float alpha) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    for (; idx < total; idx += step) {
        const long n = idx / inter;
        const int i = (int)(idx - n * inter);
        out[idx] = tw_from_float<T>(tw_glu(tw_to_float(gate_up[n * 2 * inter + i]), tw_to_float(gate_up[n * 2 * inter + inter + i]),
                                           glu, limit, alpha));
    }
}

TW_EXPORT int tw_glu_rows(void* out, const void* gate_up, int rows, int inter, int glu, float limit, float alpha, int dtype,
                          cudaStream_t stream) {
    if (rows <= 0 || inter <= 0) return 0;
    const long total = (long)rows * inter;
    const int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
    if (dtype == TW_F32)
        return tw_launch(glu_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, (float*)out, (const float*)gate_up, inter,
                         total, glu, limit, alpha);
    return tw_launch(glu_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)gate_up, inter, total, glu, limit, alpha);
}
