// Bandwidth-bound kernels: embedding gather, LayerNorm, softmax, arg-max, type conversion, weight re-layout,
// patch extraction and the small element-wise helpers.  All use 128-bit loads/stores where the row width
// and the pointers allow it and fall back to scalar accesses otherwise.
#include "common.cuh"

namespace {

constexpr int kWarp = 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Round a float32 to the nearest TF32 value (10-bit mantissa, ties to even), result kept in float32 storage.
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;   // inf / nan unchanged
    u += 0x00000fffu + ((u >> 13) & 1u);
    u &= 0xffffe000u;
    return __uint_as_float(u);
}

template <int KIND>
__device__ __forceinline__ void store4(void* out, long long idx, float4 v) {
    if constexpr (KIND == TL_OUT_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + idx) = v;
    } else if constexpr (KIND == TL_OUT_TF32) {
        float4 r = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + idx) = r;
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
        __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
        uint2 p;
        p.x = *reinterpret_cast<uint32_t*>(&a);
        p.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + idx) = p;
    }
}
template <int KIND>
__device__ __forceinline__ void store1(void* out, long long idx, float v) {
    if constexpr (KIND == TL_OUT_F32) reinterpret_cast<float*>(out)[idx] = v;
    else if constexpr (KIND == TL_OUT_TF32) reinterpret_cast<float*>(out)[idx] = round_tf32(v);
    else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

// ---- embedding gather -------------------------------------------------------------------------------
// One warp per token row: out[row,:] = table[id,:] + pos[t,:].  The single float add is exact, so the result
// is bit-identical to the NumPy path.
template <bool VEC>
__global__ void embed_kernel(const void* __restrict__ ids, int ids_type, const float* __restrict__ table,
                             const float* __restrict__ pos, float* __restrict__ out, long long rows, int T, int d,
                             int vocab, tlnn_dev_err* err) {
    long long row = (long long)blockIdx.x * (blockDim.x / kWarp) + threadIdx.x / kWarp;
    int lane = threadIdx.x % kWarp;
    if (row >= rows) return;
    long long id;
    if (ids_type == TLNN_I32) id = reinterpret_cast<const int32_t*>(ids)[row];
    else if (ids_type == TLNN_I64) id = reinterpret_cast<const int64_t*>(ids)[row];
    else id = reinterpret_cast<const uint8_t*>(ids)[row];
    if (id < 0) id += vocab;
    if (id < 0 || id >= vocab) {
        if (lane == 0) tl_dev_fail(err, TLNN_ERR_INDEX, 1, id < 0 ? id - vocab : id);
        id = 0;
    }
    int t = (int)(row % T);
    const float* src = table + id * d;
    const float* p = pos + (long long)t * d;
    float* dst = out + row * d;
    if constexpr (VEC) {
        for (int c = lane * 4; c < d; c += kWarp * 4) {
            float4 a = __ldg(reinterpret_cast<const float4*>(src + c));
            float4 b = __ldg(reinterpret_cast<const float4*>(p + c));
            float4 r = make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
            *reinterpret_cast<float4*>(dst + c) = r;
        }
    } else {
        for (int c = lane; c < d; c += kWarp) dst[c] = __fadd_rn(src[c], p[c]);
    }
}

// ---- LayerNorm -----------------------------------------------------------------------------------------
// One warp per row, the row held in registers (up to 32 x float4 per lane, d <= 4096): mean, then the mean of
// squared deviations (the two-pass form NumPy's var uses), then (x - mean) / sqrt(var + eps) * gamma + beta.
// EARLY (a few rows, as in a decode step, where the kernel is pure latency): gamma and beta, which no predecessor
// kernel writes, are loaded before the grid-dependency wait, so their latency overlaps the predecessor's tail.
template <int KIND, int VPL /* float4 per lane */, bool EARLY = false>
__global__ void layernorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                      const float* __restrict__ beta, float eps, void* __restrict__ out,
                                      long long rows, int d) {
    long long row = (long long)blockIdx.x * (blockDim.x / kWarp) + threadIdx.x / kWarp;
    int lane = threadIdx.x % kWarp;
    int nvec = d / 4;
    float4 ge[EARLY ? VPL : 1], be[EARLY ? VPL : 1];
    if (EARLY) {
        tl_grid_dependency_trigger();
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            int c = i * kWarp + lane;
            if (c < nvec) {
                ge[i] = __ldg(reinterpret_cast<const float4*>(gamma) + c);
                be[i] = __ldg(reinterpret_cast<const float4*>(beta) + c);
            }
        }
        tl_grid_dependency_wait();
    } else {
        tl_grid_dependency_sync();
    }
    if (row >= rows) return;
    const float4* src = reinterpret_cast<const float4*>(x + row * d);
    float4 v[VPL];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        int c = i * kWarp + lane;
        if (c < nvec) {
            v[i] = src[c];
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        } else {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float mean = warp_sum(s) / (float)d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        int c = i * kWarp + lane;
        if (c < nvec) {
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
        }
    }
    float var = warp_sum(q) / (float)d;
    float stdv = sqrtf(var + eps);
    const float inv = 1.f / stdv;
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    const float4* b4 = reinterpret_cast<const float4*>(beta);
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        int c = i * kWarp + lane;
        if (c < nvec) {
            float4 g, b;
            if (EARLY) { g = ge[i]; b = be[i]; }
            else { g = __ldg(g4 + c); b = __ldg(b4 + c); }
            float4 r;
            if (KIND == TL_OUT_BF16) {
                // the result is rounded to 8 significant bits: one division per row and a multiplication per
                // element instead of a division per element (which made the kernel issue-bound)
                r.x = g.x * (v[i].x * inv) + b.x;
                r.y = g.y * (v[i].y * inv) + b.y;
                r.z = g.z * (v[i].z * inv) + b.z;
                r.w = g.w * (v[i].w * inv) + b.w;
            } else {
                r.x = g.x * (v[i].x / stdv) + b.x;
                r.y = g.y * (v[i].y / stdv) + b.y;
                r.z = g.z * (v[i].z / stdv) + b.z;
                r.w = g.w * (v[i].w / stdv) + b.w;
            }
            store4<KIND>(out, row * d + c * 4, r);
        }
    }
}

// Any width: one block per row, three passes over the row (second and third hit L1/L2).
template <int KIND>
__global__ void layernorm_block_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                       const float* __restrict__ beta, float eps, void* __restrict__ out,
                                       long long rows, int d) {
    __shared__ float red[32];
    __shared__ float bcast;
    long long row = blockIdx.x;
    const float* src = x + row * d;
    int lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp, nwarp = blockDim.x / kWarp;
    auto block_sum = [&](float v) {
        v = warp_sum(v);
        if (lane == 0) red[warp] = v;
        __syncthreads();
        if (warp == 0) {
            float t = lane < nwarp ? red[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) bcast = t;
        }
        __syncthreads();
        float r = bcast;
        __syncthreads();
        return r;
    };
    float s = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) s += src[c];
    float mean = block_sum(s) / (float)d;
    float q = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { float t = src[c] - mean; q += t * t; }
    float var = block_sum(q) / (float)d;
    float stdv = sqrtf(var + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x)
        store1<KIND>(out, row * d + c, gamma[c] * ((src[c] - mean) / stdv) + beta[c]);
}

// ---- strided float32 -> {bf16, tf32-rounded, f32} copy -------------------------------------------------
template <int KIND>
__global__ void convert_kernel(const float* __restrict__ x, long long ldx, void* __restrict__ out, long long rows,
                               int cols, bool vec) {
    long long total4 = rows * (long long)(cols / 4);
    long long stride = (long long)gridDim.x * blockDim.x;
    long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        int c4 = cols / 4;
        for (long long i = i0; i < total4; i += stride) {
            long long r = i / c4;
            int c = (int)(i % c4) * 4;
            float4 v = *reinterpret_cast<const float4*>(x + r * ldx + c);
            store4<KIND>(out, r * cols + c, v);
        }
    } else {
        long long total = rows * (long long)cols;
        for (long long i = i0; i < total; i += stride) {
            long long r = i / cols;
            int c = (int)(i % cols);
            store1<KIND>(out, i, x[r * ldx + c]);
        }
    }
}

// ---- weight transpose + convert: (rows, cols) float32 -> (cols, rows) of KIND --------------------------------
template <int KIND>
__global__ void transpose_convert_kernel(const float* __restrict__ w, int rows, int cols, void* __restrict__ out) {
    __shared__ float tile[32][33];
    int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        int r = r0 + j, c = c0 + threadIdx.x;
        tile[j][threadIdx.x] = (r < rows && c < cols) ? w[(long long)r * cols + c] : 0.f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        int c = c0 + j, r = r0 + threadIdx.x;
        if (c < cols && r < rows) store1<KIND>(out, (long long)c * rows + r, tile[threadIdx.x][j]);
    }
}

// ---- softmax with temperature ----------------------------------------------------------------------------
// One block per row.  Pass 1 finds the maximum, pass 2 the sum of exp((x - max) / T), pass 3 writes; the row
// (up to ~200 KB) stays in L2 between the passes, so DRAM sees one read and one write.
__global__ void softmax_kernel(const float* __restrict__ x, float* __restrict__ out, int cols, float temperature) {
    __shared__ float red[32];
    __shared__ float bcast;
    tl_grid_dependency_sync();
    const float* src = x + (long long)blockIdx.x * cols;
    float* dst = out + (long long)blockIdx.x * cols;
    int lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp, nwarp = blockDim.x / kWarp;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, src[c]);
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    m = bcast;
    __syncthreads();
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += expf((src[c] - m) / temperature);
    s = warp_sum(s);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    s = bcast;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = expf((src[c] - m) / temperature) / s;
}

// Rows of up to 65536 values are held in the registers of one block of 1024 threads (up to 64 values per thread): every
// load of the row is in flight at once, the row is read from memory once and written once, and the exponentials are
// computed once.  exp((x - max) / T) is evaluated as 2^((x - max) * log2(e) / T) with the hardware exponential (a few
// float32 ulp from the reference's exp); the division by the row sum is a multiplication by its reciprocal.
template <int PER>
__global__ void __launch_bounds__(1024, 1) softmax_row_in_regs_kernel(const float* __restrict__ x, float* __restrict__ out, int cols, float temperature) {
    __shared__ float red[32];
    __shared__ float bcast;
    tl_grid_dependency_sync();
    const float* src = x + (long long)blockIdx.x * cols;
    float* dst = out + (long long)blockIdx.x * cols;
    const int lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp;
    float v[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int c = threadIdx.x + i * 1024;
        v[i] = c < cols ? __ldcs(src + c) : -INFINITY;       // streamed: nothing reads the input again
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; i++) m = fmaxf(m, v[i]);
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (warp == 0) {
        float t = warp_max(red[lane]);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    m = bcast;
    __syncthreads();
    const float k = 1.4426950408889634f / temperature;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        v[i] = exp2f((v[i] - m) * k);                        // 0 for the padding past the row
        s += v[i];
    }
    s = warp_sum(s);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (warp == 0) {
        float t = warp_sum(red[lane]);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    const float inv = 1.f / bcast;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int c = threadIdx.x + i * 1024;
        if (c < cols) __stcs(dst + c, v[i] * inv);
    }
}

// ---- arg-max ---------------------------------------------------------------------------------------------
// First index of the maximum, as numpy.argmax.  NaN handling: NumPy returns the first NaN; logits here are
// finite, and a NaN row yields the first maximum among the comparable values.
__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__global__ void argmax_kernel(const float* __restrict__ x, long long ldx, int32_t* __restrict__ out, int cols) {
    __shared__ float rv[32];
    __shared__ int ri[32];
    const float* src = x + (long long)blockIdx.x * ldx;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    // eight loads in flight per thread; values are combined in column order, so the first maximum wins as before
    for (int c0 = threadIdx.x; c0 < cols; c0 += blockDim.x * 8) {
        float t[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int c = c0 + u * blockDim.x;
            t[u] = c < cols ? __ldcs(src + c) : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int c = c0 + u * blockDim.x;
            if (c < cols) argmax_combine(v, idx, t[u], c);
        }
    }
    int lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp, nwarp = blockDim.x / kWarp;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_combine(v, idx, ov, oi);
    }
    if (lane == 0) { rv[warp] = v; ri[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < nwarp ? rv[lane] : -INFINITY;
        idx = lane < nwarp ? ri[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, v, o);
            int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_combine(v, idx, ov, oi);
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

// Reduce the per-tile (max, index) pairs a GEMM epilogue left behind: one warp per row.
__global__ void argmax_partials_kernel(const float2* __restrict__ parts, int n_parts, int32_t* __restrict__ out,
                                       long long rows) {
    tl_grid_dependency_sync();
    long long row = (long long)blockIdx.x * (blockDim.x / kWarp) + threadIdx.x / kWarp;
    int lane = threadIdx.x % kWarp;
    if (row >= rows) return;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int p = lane; p < n_parts; p += kWarp) {
        float2 e = parts[row * n_parts + p];
        argmax_combine(v, idx, e.x, __float_as_int(e.y));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_combine(v, idx, ov, oi);
    }
    if (lane == 0) out[row] = idx == 0x7fffffff ? 0 : idx;
}

// ---- element-wise helpers -----------------------------------------------------------------------------------
__global__ void axpby_kernel(float* __restrict__ x, float alpha, const float* __restrict__ y, float beta, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = alpha == 0.f ? 0.f : x[i] * alpha;    // alpha 0 is "fill": do not propagate old NaNs
        if (y) v += beta * y[i];
        else v += beta;
        x[i] = v;
    }
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = a[i] + b[i];
}

__global__ void gather_kernel(const float* __restrict__ src, const int64_t* __restrict__ index,
                              float* __restrict__ dst, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[index[i]];
}

__global__ void activation_kernel(int act, const float* __restrict__ x, float* __restrict__ out, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = x[i], r;
        if (act == TLNN_ACT_GELU) {
            float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
            r = 0.5f * v * (1.f + tanhf(u));
        } else if (act == TLNN_ACT_SILU) {
            r = v * ((1.f + tanhf(v * 0.5f)) * 0.5f);
        } else if (act == TLNN_ACT_RELU) {
            r = fmaxf(v, 0.f);
        } else {
            r = v;
        }
        out[i] = r;
    }
}

int grid_for(size_t n, int block, int sm_count) {
    size_t g = (n + block - 1) / block;
    size_t cap = (size_t)sm_count * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// ---- host launchers ---------------------------------------------------------------------------------------------
int tl_embed(tlnn_ctx* ctx, const void* ids, int ids_type, const float* table, const float* pos, float* out,
             int B, int T, int d, int vocab) {
    long long rows = (long long)B * T;
    if (rows == 0) return TLNN_OK;
    const int warps = 8;
    unsigned grid = (unsigned)((rows + warps - 1) / warps);
    bool vec = (d % 4 == 0) && aligned16(table) && aligned16(pos) && aligned16(out);
    if (vec)
        TL_LAUNCH(ctx, "embed_gather", embed_kernel<true><<<grid, warps * 32, 0, ctx->stream>>>(
                      ids, ids_type, table, pos, out, rows, T, d, vocab, ctx->d_err));
    else
        TL_LAUNCH(ctx, "embed_gather", embed_kernel<false><<<grid, warps * 32, 0, ctx->stream>>>(
                      ids, ids_type, table, pos, out, rows, T, d, vocab, ctx->d_err));
    return TLNN_OK;
}

template <int KIND>
static int layernorm_dispatch(tlnn_ctx* ctx, const float* x, const float* gamma, const float* beta, float eps,
                              void* out, long long rows, int d) {
    bool vec = (d % 4 == 0) && d <= 4096 && aligned16(x) && aligned16(gamma) && aligned16(beta) && aligned16(out);
    if (vec) {
        const int warps = 4;
        unsigned grid = (unsigned)((rows + warps - 1) / warps);
        int vpl = (d / 4 + 31) / 32;
#define LN_CASE(V)                                                                                              \
    TL_LAUNCH(ctx, "layernorm", tl_launch_kernel(ctx, layernorm_warp_kernel<KIND, V>, dim3(grid), dim3(warps * 32), 0, \
                                                 x, gamma, beta, eps, out, rows, d))
#define LN_EARLY(V)                                                                                             \
    TL_LAUNCH(ctx, "layernorm", tl_launch_kernel(ctx, layernorm_warp_kernel<KIND, V, true>, dim3(grid), dim3(warps * 32), 0, \
                                                 x, gamma, beta, eps, out, rows, d))
        if (rows <= 1024 && vpl <= 8) {
            if (vpl <= 2) LN_EARLY(2);
            else if (vpl <= 4) LN_EARLY(4);
            else if (vpl <= 6) LN_EARLY(6);
            else LN_EARLY(8);
        }
        else if (vpl <= 1) LN_CASE(1);
        else if (vpl <= 2) LN_CASE(2);
        else if (vpl <= 4) LN_CASE(4);
        else if (vpl <= 6) LN_CASE(6);
        else if (vpl <= 8) LN_CASE(8);
        else if (vpl <= 16) LN_CASE(16);
        else LN_CASE(32);
#undef LN_CASE
#undef LN_EARLY
    } else {
        TL_LAUNCH(ctx, "layernorm", layernorm_block_kernel<KIND><<<(unsigned)rows, 256, 0, ctx->stream>>>(
                      x, gamma, beta, eps, out, rows, d));
    }
    return TLNN_OK;
}

int tl_layernorm(tlnn_ctx* ctx, const float* x, const float* gamma, const float* beta, float eps, void* out,
                 int out_kind, long long rows, int d) {
    if (rows == 0) return TLNN_OK;
    TL_REQUIRE(rows < (1ll << 31), "too many rows");
    if (out_kind == TL_OUT_F32) return layernorm_dispatch<TL_OUT_F32>(ctx, x, gamma, beta, eps, out, rows, d);
    if (out_kind == TL_OUT_BF16) return layernorm_dispatch<TL_OUT_BF16>(ctx, x, gamma, beta, eps, out, rows, d);
    return layernorm_dispatch<TL_OUT_TF32>(ctx, x, gamma, beta, eps, out, rows, d);
}

int tl_convert(tlnn_ctx* ctx, const float* x, long long ldx, void* out, int out_kind, long long rows, int cols) {
    if (rows == 0 || cols == 0) return TLNN_OK;
    bool vec = (cols % 4 == 0) && (ldx % 4 == 0) && aligned16(x) && aligned16(out);
    size_t n = (size_t)rows * cols / (vec ? 4 : 1);
    int grid = grid_for(n, 256, ctx->sm_count);
    if (out_kind == TL_OUT_BF16)
        TL_LAUNCH(ctx, "convert", convert_kernel<TL_OUT_BF16><<<grid, 256, 0, ctx->stream>>>(x, ldx, out, rows, cols, vec));
    else if (out_kind == TL_OUT_TF32)
        TL_LAUNCH(ctx, "convert", convert_kernel<TL_OUT_TF32><<<grid, 256, 0, ctx->stream>>>(x, ldx, out, rows, cols, vec));
    else
        TL_LAUNCH(ctx, "convert", convert_kernel<TL_OUT_F32><<<grid, 256, 0, ctx->stream>>>(x, ldx, out, rows, cols, vec));
    return TLNN_OK;
}

int tl_argmax_partials(tlnn_ctx* ctx, const float2* partials, int n_parts, int32_t* tokens, long long rows) {
    if (rows == 0) return TLNN_OK;
    const int warps = 8;
    unsigned grid = (unsigned)((rows + warps - 1) / warps);
    TL_LAUNCH(ctx, "argmax_partials",
              tl_launch_kernel(ctx, argmax_partials_kernel, dim3(grid), dim3(warps * 32), 0, partials, n_parts, tokens, rows));
    return TLNN_OK;
}

// ---- C ABI ---------------------------------------------------------------------------------------------------------
extern "C" int tlnn_embed_fwd(tlnn_ctx* ctx, const void* ids, int ids_type, const float* table, const float* pos,
                              float* out, int B, int T, int d, int vocab) {
    TL_NOTNULL(ctx); TL_NOTNULL(ids); TL_NOTNULL(table); TL_NOTNULL(pos); TL_NOTNULL(out);
    TL_REQUIRE(B >= 0 && T >= 0 && d > 0 && vocab > 0, "embed: bad shape B=%d T=%d d=%d vocab=%d", B, T, d, vocab);
    TL_REQUIRE(ids_type == TLNN_I32 || ids_type == TLNN_I64 || ids_type == TLNN_U8,
               "embed: token ids must be int32, int64 or uint8");
    TL_CUDA(cudaSetDevice(ctx->device));
    return tl_embed(ctx, ids, ids_type, table, pos, out, B, T, d, vocab);
}

extern "C" int tlnn_layernorm_fwd(tlnn_ctx* ctx, const float* x, const float* gamma, const float* beta, float eps,
                                  float* out, long long rows, int d) {
    TL_NOTNULL(ctx); TL_NOTNULL(x); TL_NOTNULL(gamma); TL_NOTNULL(beta); TL_NOTNULL(out);
    TL_REQUIRE(rows >= 0 && d > 0, "layernorm: bad shape rows=%lld d=%d", rows, d);
    TL_CUDA(cudaSetDevice(ctx->device));
    return tl_layernorm(ctx, x, gamma, beta, eps, out, TL_OUT_F32, rows, d);
}

extern "C" int tlnn_activation_fwd(tlnn_ctx* ctx, int act, const float* x, float* out, size_t n) {
    TL_NOTNULL(ctx);
    TL_REQUIRE(act >= TLNN_ACT_NONE && act <= TLNN_ACT_RELU, "unknown activation %d", act);
    if (n == 0) return TLNN_OK;
    TL_NOTNULL(x); TL_NOTNULL(out);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_LAUNCH(ctx, "activation", activation_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(act, x, out, n));
    return TLNN_OK;
}

extern "C" int tlnn_softmax_fwd(tlnn_ctx* ctx, const float* x, float* out, long long rows, int cols, float temperature) {
    TL_NOTNULL(ctx);
    TL_REQUIRE(rows >= 0 && cols > 0 && rows < (1ll << 31), "softmax: bad shape rows=%lld cols=%d", rows, cols);
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(x); TL_NOTNULL(out);
    TL_CUDA(cudaSetDevice(ctx->device));
    int block = cols >= 8192 ? 1024 : (cols >= 1024 ? 256 : 64);
    if (cols > 4096 && cols <= 65536) {
        // wide rows (a vocabulary): the row in the registers of one block, one read and one write
        const int per = (cols + 1023) / 1024;
        if (per <= 16) TL_LAUNCH(ctx, "softmax", tl_launch_kernel(ctx, softmax_row_in_regs_kernel<16>, dim3((unsigned)rows), dim3(1024), 0, x, out, cols, temperature));
        else if (per <= 32) TL_LAUNCH(ctx, "softmax", tl_launch_kernel(ctx, softmax_row_in_regs_kernel<32>, dim3((unsigned)rows), dim3(1024), 0, x, out, cols, temperature));
        else if (per <= 50) TL_LAUNCH(ctx, "softmax", tl_launch_kernel(ctx, softmax_row_in_regs_kernel<50>, dim3((unsigned)rows), dim3(1024), 0, x, out, cols, temperature));
        else TL_LAUNCH(ctx, "softmax", tl_launch_kernel(ctx, softmax_row_in_regs_kernel<64>, dim3((unsigned)rows), dim3(1024), 0, x, out, cols, temperature));
        return TLNN_OK;
    }
    TL_LAUNCH(ctx, "softmax", tl_launch_kernel(ctx, softmax_kernel, dim3((unsigned)rows), dim3(block), 0, x, out, cols, temperature));
    return TLNN_OK;
}

namespace {
// Inverse-CDF draw, one block per row.  Thread t owns the contiguous segment t of the row: segment sums (double),
// an exclusive scan of the 256 sums, then the thread whose segment holds the target walks it.  The comparison is
// NumPy's: prefix / total > u.
// The uniform number of row r is uniforms[step * rows + r], with the step read from device memory when given (a
// decode step captured in a CUDA graph advances it on the device).
__global__ void __launch_bounds__(256) sample_kernel(const float* __restrict__ probs, long long ldp, const double* __restrict__ uniforms,
                                                     const int* __restrict__ step, int32_t* __restrict__ out, int cols) {
    __shared__ double seg[256];
    __shared__ int found;
    tl_grid_dependency_sync();
    const long long row = blockIdx.x;
    const float* p = probs + row * ldp;
    const int per = (cols + 255) / 256;
    const int lo = min(cols, (int)threadIdx.x * per), hi = min(cols, lo + per);
    double s = 0.0;
    for (int i = lo; i < hi; i++) s += (double)p[i];
    seg[threadIdx.x] = s;
    if (threadIdx.x == 0) found = cols - 1;          // u so close to 1 that no prefix exceeds it: the last index
    __syncthreads();
    double before = 0.0, total = 0.0;
    for (int t = 0; t < 256; t++) {
        if (t == (int)threadIdx.x) before = total;
        total += seg[t];
    }
    const double u = uniforms[(step ? (long long)*step * gridDim.x : 0ll) + row];
    double c = before;
    int mine = cols;
    for (int i = lo; i < hi; i++) {
        c += (double)p[i];
        if (c / total > u) { mine = i; break; }
    }
    if (mine < cols) atomicMin(&found, mine);
    __syncthreads();
    if (threadIdx.x == 0) out[row] = found;
}
}  // namespace

int tl_sample(tlnn_ctx* ctx, const float* probs, long long ldp, const double* uniforms, const int* step, int32_t* out,
              long long rows, int cols) {
    TL_LAUNCH(ctx, "sample", tl_launch_kernel(ctx, sample_kernel, dim3((unsigned)rows), dim3(256), 0, probs, ldp, uniforms, step, out, cols));
    return TLNN_OK;
}

extern "C" int tlnn_sample_fwd(tlnn_ctx* ctx, const float* probs, long long ldp, const double* uniforms, int32_t* out,
                               long long rows, int cols) {
    TL_NOTNULL(ctx);
    TL_REQUIRE(rows >= 0 && cols > 0 && rows < (1ll << 31) && ldp >= cols, "sample: bad shape rows=%lld cols=%d", rows, cols);
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(probs); TL_NOTNULL(uniforms); TL_NOTNULL(out);
    TL_CUDA(cudaSetDevice(ctx->device));
    return tl_sample(ctx, probs, ldp, uniforms, nullptr, out, rows, cols);
}

namespace {
__device__ __forceinline__ long long label_at(const void* labels, int type, long long i) {
    if (type == TLNN_I32) return reinterpret_cast<const int32_t*>(labels)[i];
    if (type == TLNN_I64) return reinterpret_cast<const long long*>(labels)[i];
    return reinterpret_cast<const uint8_t*>(labels)[i];
}

// One block per row: first index of the row maximum against the label, and the row's cross-entropy term.
__global__ void __launch_bounds__(256) eval_batch_kernel(const float* __restrict__ probs, long long ldp, const void* __restrict__ labels,
                                                         int labels_type, int cols, double* loss_sum, unsigned long long* correct,
                                                         tlnn_dev_err* err) {
    __shared__ float best_v[256];
    __shared__ int best_i[256];
    const long long row = blockIdx.x;
    const float* p = probs + row * ldp;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = p[i];
        if (v > bv) { bv = v; bi = i; }           // strided scan keeps the smallest index of a thread's maximum
    }
    best_v[threadIdx.x] = bv; best_i[threadIdx.x] = bi;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) {
            const float ov = best_v[threadIdx.x + s];
            const int oi = best_i[threadIdx.x + s];
            if (ov > best_v[threadIdx.x] || (ov == best_v[threadIdx.x] && oi < best_i[threadIdx.x])) {
                best_v[threadIdx.x] = ov; best_i[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const long long label = label_at(labels, labels_type, row);
        if (label < 0 || label >= cols) {
            tl_dev_fail(err, TLNN_ERR_INDEX, 301, label);
            return;
        }
        atomicAdd(loss_sum, (double)(-logf(p[label] + 1e-7f)));
        if (best_i[0] == (int)label) atomicAdd(correct, 1ull);
    }
}
}  // namespace

extern "C" int tlnn_eval_batch_fwd(tlnn_ctx* ctx, const float* probs, long long ldp, const void* labels, int labels_type,
                                   long long rows, int cols, double* loss_sum, long long* correct) {
    TL_NOTNULL(ctx);
    TL_REQUIRE(rows >= 0 && cols > 0 && rows < (1ll << 31) && ldp >= cols, "eval: bad shape rows=%lld cols=%d", rows, cols);
    TL_REQUIRE(labels_type == TLNN_I32 || labels_type == TLNN_I64 || labels_type == TLNN_U8, "eval: labels must be int32, int64 or uint8");
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(probs); TL_NOTNULL(labels); TL_NOTNULL(loss_sum); TL_NOTNULL(correct);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_LAUNCH(ctx, "eval_batch", eval_batch_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(
                  probs, ldp, labels, labels_type, cols, loss_sum, reinterpret_cast<unsigned long long*>(correct), ctx->d_err));
    return TLNN_OK;
}

extern "C" int tlnn_argmax_fwd(tlnn_ctx* ctx, const float* x, long long ldx, int32_t* out, long long rows, int cols) {
    TL_NOTNULL(ctx);
    TL_REQUIRE(rows >= 0 && cols > 0 && rows < (1ll << 31) && ldx >= cols, "argmax: bad shape rows=%lld cols=%d", rows, cols);
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(x); TL_NOTNULL(out);
    TL_CUDA(cudaSetDevice(ctx->device));
    int block = cols >= 8192 ? 1024 : (cols >= 1024 ? 256 : 64);
    TL_LAUNCH(ctx, "argmax", argmax_kernel<<<(unsigned)rows, block, 0, ctx->stream>>>(x, ldx, out, cols));
    return TLNN_OK;
}

extern "C" int tlnn_axpby_f32(tlnn_ctx* ctx, float* x, float alpha, const float* y, float beta, size_t n) {
    TL_NOTNULL(ctx);
    if (n == 0) return TLNN_OK;
    TL_NOTNULL(x);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_LAUNCH(ctx, "axpby", axpby_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(x, alpha, y, beta, n));
    return TLNN_OK;
}

extern "C" int tlnn_add_f32(tlnn_ctx* ctx, const float* a, const float* b, float* out, size_t n) {
    TL_NOTNULL(ctx);
    if (n == 0) return TLNN_OK;
    TL_NOTNULL(a); TL_NOTNULL(b); TL_NOTNULL(out);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_LAUNCH(ctx, "add", add_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(a, b, out, n));
    return TLNN_OK;
}

extern "C" int tlnn_gather_f32(tlnn_ctx* ctx, const float* src, const int64_t* index, float* dst, size_t n) {
    TL_NOTNULL(ctx);
    if (n == 0) return TLNN_OK;
    TL_NOTNULL(src); TL_NOTNULL(index); TL_NOTNULL(dst);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_LAUNCH(ctx, "gather", gather_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(src, index, dst, n));
    return TLNN_OK;
}

extern "C" int tlnn_weight_prepare(tlnn_ctx* ctx, const float* w, int rows, int cols, int transpose, int prec, void* out) {
    TL_NOTNULL(ctx); TL_NOTNULL(w); TL_NOTNULL(out);
    TL_REQUIRE(rows > 0 && cols > 0, "weight_prepare: bad shape %d x %d", rows, cols);
    TL_REQUIRE(prec == TLNN_PREC_TF32 || prec == TLNN_PREC_BF16, "weight_prepare: unknown precision %d", prec);
    TL_CUDA(cudaSetDevice(ctx->device));
    int kind = prec == TLNN_PREC_BF16 ? TL_OUT_BF16 : TL_OUT_TF32;
    if (!transpose) return tl_convert(ctx, w, cols, out, kind, rows, cols);
    dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
    if (kind == TL_OUT_BF16)
        TL_LAUNCH(ctx, "weight_transpose", transpose_convert_kernel<TL_OUT_BF16><<<grid, block, 0, ctx->stream>>>(w, rows, cols, out));
    else
        TL_LAUNCH(ctx, "weight_transpose", transpose_convert_kernel<TL_OUT_TF32><<<grid, block, 0, ctx->stream>>>(w, rows, cols, out));
    return TLNN_OK;
}
