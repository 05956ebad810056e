// Row kernels of blocks that normalise a sublayer's result before it joins the stream, and two activations:
//
//   gated_norm_add   y = d * sigmoid(g + bias) (the gate is optional);  x <- x + rms(y) * w;  optionally the new
//                    rows once more in the compute dtype, and the NEXT norm of the new rows, rms(x) * w2
//   polynorm_rows    out = a rms(z) + b rms(z^2) + c rms(z^3) + e  over a row of a product
//   softcap_rows     z <- cap tanh(z / cap), in place
//
// rms(y) = y / sqrt(mean(y^2) + eps).  Products arrive as float32, possibly as split-K parts that are summed in
// order; every sum and every norm is float32.
#include <algorithm>

#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {

__device__ __forceinline__ float load_parts(const float* p, size_t idx, int nsplit, size_t stride) {
    float v = p[idx];
#pragma unroll 4
    for (int s = 1; s < nsplit; ++s) v += p[idx + (size_t)s * stride];
    return v;
}

// four neighbours at once: the parts' loads of a thread are all in flight before the first addition
__device__ __forceinline__ float4 load_parts4(const float* p, size_t idx, int nsplit, size_t stride) {
    float4 v = *reinterpret_cast<const float4*>(p + idx);
#pragma unroll 8
    for (int s = 1; s < nsplit; ++s) {
        const float4 u = *reinterpret_cast<const float4*>(p + idx + (size_t)s * stride);
        v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
    }
    return v;
}
__device__ __forceinline__ void store4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float4& v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float sigmoid_(float z) { return 1.f / (1.f + expf(-z)); }

// VEC: H, the parts' strides and g's row stride are multiples of 4 and every pointer sits on 16 bytes (8 for bfloat16)
template <typename CT, bool VEC>
__global__ void __launch_bounds__(1024)
gated_norm_add_kernel(float* __restrict__ x, const float* __restrict__ d, int dn, size_t ds,
                      const float* __restrict__ g, int gn, size_t gs, int g_ld, const float* __restrict__ bias,
                      const float* __restrict__ w, float eps, CT* __restrict__ copy,
                      const float* __restrict__ w2, float eps2, CT* __restrict__ next, int H) {
    extern __shared__ __align__(16) float row[];       // y, then the new x
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    float ss = 0.f, s2 = 0.f;
    if (VEC) {
        for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
            float4 y = load_parts4(d, r * H + i, dn, ds);
            if (g) {
                float4 z = load_parts4(g, r * g_ld + i, gn, gs);
                if (bias) {
                    const float4 bb = *reinterpret_cast<const float4*>(bias + i);
                    z.x += bb.x; z.y += bb.y; z.z += bb.z; z.w += bb.w;
                }
                y.x *= sigmoid_(z.x); y.y *= sigmoid_(z.y); y.z *= sigmoid_(z.z); y.w *= sigmoid_(z.w);
            }
            store4(row + i, y);
            ss += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float y = load_parts(d, r * H + i, dn, ds);
            if (g) y *= sigmoid_(load_parts(g, r * g_ld + i, gn, gs) + (bias ? bias[i] : 0.f));
            row[i] = y;
            ss += y * y;
        }
    }
    const float rinv = 1.f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    if (VEC) {
        for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
            const float4 y = *reinterpret_cast<const float4*>(row + i), ww = *reinterpret_cast<const float4*>(w + i);
            float4 v = *reinterpret_cast<const float4*>(x + r * H + i);
            v.x += y.x * rinv * ww.x; v.y += y.y * rinv * ww.y; v.z += y.z * rinv * ww.z; v.w += y.w * rinv * ww.w;
            store4(x + r * H + i, v);
            store4(row + i, v);
            if (copy) store4(copy + r * H + i, v);
            s2 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = x[r * H + i] + row[i] * rinv * w[i];
            x[r * H + i] = v;
            row[i] = v;
            if (copy) copy[r * H + i] = from_float<CT>(v);
            s2 += v * v;
        }
    }
    if (!next) return;
    const float rinv2 = 1.f / sqrtf(block_sum(s2, scratch) / (float)H + eps2);
    if (VEC) {
        for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(row + i), ww = *reinterpret_cast<const float4*>(w2 + i);
            store4(next + r * H + i, make_float4(v.x * rinv2 * ww.x, v.y * rinv2 * ww.y, v.z * rinv2 * ww.z, v.w * rinv2 * ww.w));
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) next[r * H + i] = from_float<CT>(row[i] * rinv2 * w2[i]);
    }
}

template <typename OT>
__global__ void __launch_bounds__(256)
polynorm_kernel(const float* __restrict__ z, int zn, size_t zs, const float* __restrict__ coef, float eps,
                OT* __restrict__ out, int F) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = load_parts(z, r * F + i, zn, zs);
        row[i] = v;
        const float v2 = v * v, v3 = v2 * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += v3 * v3;
    }
    const float r1 = 1.f / sqrtf(block_sum(s1, scratch) / (float)F + eps);
    const float r2 = 1.f / sqrtf(block_sum(s2, scratch) / (float)F + eps);
    const float r3 = 1.f / sqrtf(block_sum(s3, scratch) / (float)F + eps);
    const float a = coef[0] * r1, b = coef[1] * r2, c = coef[2] * r3, e = coef[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = row[i], v2 = v * v;
        out[r * F + i] = from_float<OT>(a * v + b * v2 + c * (v2 * v) + e);
    }
}

__global__ void softcap_kernel(float* __restrict__ z, float cap, float inv_cap, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        z[i] = cap * tanhf(z[i] * inv_cap);
}

constexpr size_t SMEM_MAX = 200 * 1024;

template <typename Kern>
int raise_smem(Kern kern, size_t smem, const char* what) {
    if (smem > SMEM_MAX) return fail("%s: a row of %zu bytes does not fit an SM's shared memory", what, smem);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX) != cudaSuccess)
        return fail("%s: cannot raise the shared-memory limit", what);
    return 0;
}

}  // namespace

MHB_EXPORT int mhb_gated_norm_add(float* x, const float* d, int dn, long long ds, const float* g, int gn, long long gs,
                                  int g_ld, const float* bias, const float* w, float eps, void* copy, const float* w2,
                                  float eps2, void* next, int out_dtype, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    const size_t smem = sizeof(float) * (size_t)H;
    auto on16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = H % 4 == 0 && ds % 4 == 0 && on16(x) && on16(d) && on16(w) && (!g || (gs % 4 == 0 && g_ld % 4 == 0 && on16(g))) &&
                     (!bias || on16(bias)) && (!copy || on16(copy)) && (!next || (on16(next) && on16(w2)));
    // a row's elements in fours over up to 1024 threads (few rows, long rows: decoded tokens wait on latency alone)
    const int per = vec ? 4 : 1, threads = std::min(1024, std::max(128, ((H + per - 1) / per + 31) / 32 * 32));
    MHB_DISPATCH_DTYPE(out_dtype, CT, {
        cudaError_t e;
        if (vec) {
            if (int rc = raise_smem(gated_norm_add_kernel<CT, true>, smem, "gated_norm_add")) return rc;
            e = launch_kernel(gated_norm_add_kernel<CT, true>, dim3(R), dim3(threads), smem, stream, x, d, dn, (size_t)ds, g,
                              gn, (size_t)gs, g_ld, bias, w, eps, (CT*)copy, w2, eps2, (CT*)next, H);
        } else {
            if (int rc = raise_smem(gated_norm_add_kernel<CT, false>, smem, "gated_norm_add")) return rc;
            e = launch_kernel(gated_norm_add_kernel<CT, false>, dim3(R), dim3(threads), smem, stream, x, d, dn, (size_t)ds, g,
                              gn, (size_t)gs, g_ld, bias, w, eps, (CT*)copy, w2, eps2, (CT*)next, H);
        }
        if (e != cudaSuccess) return fail("gated_norm_add: %s", cudaGetErrorString(e));
    });
    return check_launch("gated_norm_add");
}

MHB_EXPORT int mhb_polynorm_rows(const float* z, int zn, long long zs, const float* coef, float eps, void* out,
                                 int out_dtype, int R, int F, cudaStream_t stream) {
    if (R <= 0) return 0;
    const size_t smem = sizeof(float) * (size_t)F;
    MHB_DISPATCH_DTYPE(out_dtype, OT, {
        if (int rc = raise_smem(polynorm_kernel<OT>, smem, "polynorm_rows")) return rc;
        cudaError_t e = launch_kernel(polynorm_kernel<OT>, dim3(R), dim3(256), smem, stream, z, zn, (size_t)zs, coef, eps,
                                      (OT*)out, F);
        if (e != cudaSuccess) return fail("polynorm_rows: %s", cudaGetErrorString(e));
    });
    return check_launch("polynorm_rows");
}

MHB_EXPORT int mhb_softcap_rows(float* z, float cap, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return fail("softcap_rows: the cap must be positive");
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    cudaError_t e = launch_kernel(softcap_kernel, dim3(blocks), dim3(256), 0, stream, z, cap, 1.f / cap, n);
    if (e != cudaSuccess) return fail("softcap_rows: %s", cudaGetErrorString(e));
    return check_launch("softcap_rows");
}
