// Row-wise kernels of the decoder: embedding gather, fused residual-add + RMSNorm, SwiGLU,
// rotary table, fused per-head q/k RMSNorm + rotation + cache write, row gather.
//
// The residual stream is float32 in both engine precisions; norms and rotation are computed
// in float32 (angles in float64, then rounded, exactly as the reference builds its table:
// crates/aien-inference-abi/src/tensor.rs:150-163).
#include "common.cuh"

namespace aien {

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ x, int H, int V) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* row = x + (size_t)t * H;
    if (id < 0 || id >= V) {                      // refused on the host; never read out of range
        for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = to_f(src[i]);
}

// ---------------------------------------------------------------- residual add + RMSNorm
// x[t] += sum_p delta[p][t] (if delta), then h[t] = x[t] * (1/sqrt(mean(x^2)+eps)) * w   (tensor.rs:94-110)
// `delta` may be `nparts` float32 partial products [nparts][T][H] (the split-K decode product
// leaves its reduction to this kernel); they are added in index order.
template <typename TD>
__device__ __forceinline__ float delta_sum(const TD* __restrict__ delta, int nparts, size_t part_stride, size_t idx) {
    float d = 0.f;
    for (int p = 0; p < nparts; ++p) d += ld_act(delta + (size_t)p * part_stride + idx);
    return d;
}

template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int nparts, size_t part_stride,
                                   const void* __restrict__ w, int wdt, float eps,
                                   TO* __restrict__ h, int H) {
    __shared__ float red[32];
    griddep_launch();
    griddep_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[base + i];
        if (delta != nullptr) {
            v += delta_sum(delta, nparts, part_stride, base + i);
            x[base + i] = v;
        }
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        h[base + i] = from_f<TO>(x[base + i] * scale * load_dyn(w, wdt, i));
    }
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 load4_dyn(const void* p, int dt, size_t i) {
    return dt == AIEN_DT_F32 ? load4(reinterpret_cast<const float*>(p) + i) : load4(reinterpret_cast<const __nv_bfloat16*>(p) + i);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

// Same, for H % 4 == 0 and H <= 256 * 4 * NV, all rows 16-byte aligned: the row stays in registers
// between the passes, every access is a vector, and all loads of a thread (the row, the pending
// sums, the weights) are issued before the first use.
// PARTS: the pending sum comes in several parts (the register budget of that case is its own).
// BS threads a row: 256, or 1,024 for steps of so few rows that the grid leaves most SMs empty; a
// thread then holds one vector of the row and has every load it makes in flight at once.
template <typename TD, typename TO, int NV, bool PARTS, int BS>
__global__ void __launch_bounds__(BS)
add_rmsnorm_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta, int nparts, size_t part_stride,
                       const void* __restrict__ w, int wdt, float eps, TO* __restrict__ h, int H) {
    __shared__ float red[32];
    griddep_launch();
    float4 wv[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {                                   // weights do not depend on the kernel ahead
        const int i = (j * BS + threadIdx.x) * 4;
        wv[j] = i < H ? load4_dyn(w, wdt, i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    griddep_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = (j * BS + threadIdx.x) * 4;
        v[j] = i < H ? load4(x + base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (delta != nullptr) {
        if (!PARTS) {
            float4 dv[NV];
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int i = (j * BS + threadIdx.x) * 4;
                dv[j] = i < H ? ld_act4(delta + base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < NV; ++j) { v[j].x += dv[j].x; v[j].y += dv[j].y; v[j].z += dv[j].z; v[j].w += dv[j].w; }
        } else {
            // four parts are requested at once (the loads of a part do not wait for the sums of the one
            // before); they are added in index order
            constexpr int PU = NV == 1 ? 8 : (NV <= 4 ? 4 : 2);
            for (int p0 = 0; p0 < nparts; p0 += PU) {
                float4 d[PU][NV];
#pragma unroll
                for (int pp = 0; pp < PU; ++pp)
#pragma unroll
                    for (int j = 0; j < NV; ++j) {
                        const int i = (j * BS + threadIdx.x) * 4;
                        if (p0 + pp < nparts && i < H) d[pp][j] = ld_act4(delta + (size_t)(p0 + pp) * part_stride + base + i);
                    }
#pragma unroll
                for (int pp = 0; pp < PU; ++pp)
                    if (p0 + pp < nparts) {
#pragma unroll
                        for (int j = 0; j < NV; ++j) {
                            const int i = (j * BS + threadIdx.x) * 4;
                            if (i < H) { v[j].x += d[pp][j].x; v[j].y += d[pp][j].y; v[j].z += d[pp][j].z; v[j].w += d[pp][j].w; }
                        }
                    }
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = (j * BS + threadIdx.x) * 4;
        if (i < H) {
            if (delta != nullptr) store4(x + base + i, v[j]);
            store4(h + base + i, make_float4(v[j].x * scale * wv[j].x, v[j].y * scale * wv[j].y,
                                             v[j].z * scale * wv[j].z, v[j].w * scale * wv[j].w));
        }
    }
}

// out[r] = x[rows[r]] + sum_p delta[p][rows[r]]   (float32 out; feeds the final norm of wanted rows only)
template <typename TD>
__global__ void gather_add_rows_kernel(const float* __restrict__ x, const TD* __restrict__ delta, int nparts,
                                       size_t part_stride, const int* __restrict__ rows, float* __restrict__ out, int H) {
    griddep_launch();
    griddep_wait();
    const size_t src = (size_t)rows[blockIdx.x] * H, dst = (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = ld_act(x + src + i);
        if (delta != nullptr) v += delta_sum(delta, nparts, part_stride, src + i);
        out[dst + i] = v;
    }
}

// x[t] += sum_p delta[p][t]   (the residual sum alone, for arrangements that do not norm right after it)
template <typename TD>
__global__ void add_residual_kernel(float* __restrict__ x, const TD* __restrict__ delta, int nparts, size_t part_stride, size_t total) {
    griddep_launch();
    griddep_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) x[idx] = ld_act(x + idx) + delta_sum(delta, nparts, part_stride, idx);
}

// ---------------------------------------------------------------- SwiGLU
// a = silu(g) * u, silu(g) = g / (1 + exp(-g))     (backend.rs:572-579).  gu = [T, 2I]:
// group == 0: gate columns [0, I), up columns [I, 2I);  group > 0: columns interleaved in runs of
// `group` (gate run, then the matching up run), the layout the fused decode product wants.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int group, size_t total) {
    griddep_launch();
    griddep_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / I, i = idx - t * I;
        size_t gi, ui;
        if (group == 0) { gi = i; ui = I + i; }
        else { gi = (i / group) * 2 * group + (i % group); ui = gi + group; }
        const float g = ld_act(gu + t * 2 * I + gi);
        const float u = ld_act(gu + t * 2 * I + ui);
        out[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
    }
}

// ---------------------------------------------------------------- rotary table
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t, int T, int half) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    double s, c;
    sincos((double)positions[t] * inv_freq[i], &s, &c);
    cos_t[idx] = (float)c;
    sin_t[idx] = (float)s;
}

// ---------------------------------------------------------------- q/k norm + rotation + cache write
// One warp per (token, head).  For a q or k head: optional RMSNorm over the head
// (tensor.rs:114-121), then rotate_half pairing (i, i + rot/2) on the first `rot` values
// (tensor.rs:165-188).  q goes to q_out (which may be q itself); k and v go to the cache slot of
// the token, rounded once to the cache dtype (crates/aien-kv-cache/src/lib.rs:88-101).
// The inputs may be `nparts` float32 partial products laid out [nparts][T][row] (split-K decode).
#define AIEN_MAX_HEAD_DIM 256
template <typename TI, typename TC, typename TKV>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_write_kernel(
    const TI* q, long q_stride, int nq,
    const TI* __restrict__ k, long k_stride, const TI* __restrict__ v, long v_stride, int nkv,
    int nparts, size_t part_stride, TC* q_out, long q_out_stride,
    int hd, const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int wdt, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
    const int* __restrict__ slot_map, TKV* __restrict__ k_cache, TKV* __restrict__ v_cache) {
    __shared__ float buf[4][AIEN_MAX_HEAD_DIM];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = rot >> 1;
    const bool write_kv = (k != nullptr);
    const int n_heads = nq + (write_kv ? 2 * nkv : 0);
    const int head = blockIdx.y * 4 + warp;
    if (head >= n_heads) return;
    const long slot = write_kv ? (long)__ldcg(slot_map + t) : -1;
    float* hb = buf[warp];
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const int hh = is_q ? head : (is_k ? head - nq : head - nq - nkv);
    if (!is_q && slot < 0) return;                               // token has no cache slot
    const TI* src = is_q ? (q + (size_t)t * q_stride + (size_t)hh * hd)
                         : (is_k ? (k + (size_t)t * k_stride + (size_t)hh * hd)
                                 : (v + (size_t)t * v_stride + (size_t)hh * hd));
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
        float val = 0.f;
        for (int p = 0; p < nparts; ++p) val += ld_act(src + (size_t)p * part_stride + i);
        hb[i] = val;
        ss += val * val;
    }
    __syncwarp();
    if (is_q || is_k) {
        const void* nw = is_q ? q_norm_w : k_norm_w;
        if (nw != nullptr) {
            ss = warp_sum(ss);
            const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
            for (int i = lane; i < hd; i += 32) hb[i] = hb[i] * scale * load_dyn(nw, wdt, i);
            __syncwarp();
        }
        if (cos_t != nullptr) {
            for (int i = lane; i < half; i += 32) {
                const float a = hb[i], b = hb[i + half];
                const float c = __ldcg(cos_t + (size_t)t * half + i), s = __ldcg(sin_t + (size_t)t * half + i);
                hb[i] = a * c - b * s;
                hb[i + half] = a * s + b * c;
            }
            __syncwarp();
        }
    }
    if (is_q) {
        TC* dst = q_out + (size_t)t * q_out_stride + (size_t)hh * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = from_f<TC>(hb[i]);
    } else {
        TKV* dst = (is_k ? k_cache : v_cache) + ((size_t)slot * nkv + hh) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = from_f<TKV>(hb[i]);
    }
}

// The same for the common case (bfloat16 everywhere, head size 128, rotation over the whole head or
// none, one input part): a warp per head, four consecutive values per lane, no shared memory.  The
// rotation partner of value i is i +- 64, which lane ^ 16 holds.  A warp takes QK_TOKENS tokens of
// its head at once, so that many independent loads are in flight; weights do not depend on the
// kernel ahead and are requested before the wait for it.
constexpr int QK_TOKENS = 4;
template <typename TI>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_write_hd128_kernel(
    const TI* q, long q_stride, int nq, const TI* __restrict__ k, long k_stride,
    const TI* __restrict__ v, long v_stride, int nkv, int nparts, size_t part_stride, __nv_bfloat16* q_out, long q_out_stride,
    const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int wdt, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int T) {
    griddep_launch();
    const int t0 = blockIdx.x * QK_TOKENS, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool write_kv = (k != nullptr);
    const int n_heads = nq + (write_kv ? 2 * nkv : 0);
    const int head = blockIdx.y * 4 + warp;
    if (head >= n_heads) return;
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const int hh = is_q ? head : (is_k ? head - nq : head - nq - nkv);
    const void* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    const bool rotate = cos_t != nullptr && (is_q || is_k);
    float4 wv = make_float4(1.f, 1.f, 1.f, 1.f);
    if (nw != nullptr) wv = load4_dyn(nw, wdt, lane * 4);
    griddep_wait();
    const TI* src_base = is_q ? q : (is_k ? k : v);
    const long src_stride = is_q ? q_stride : (is_k ? k_stride : v_stride);
    long slot[QK_TOKENS];
    float4 raw[QK_TOKENS];
    float4 cs[QK_TOKENS], sn[QK_TOKENS];
#pragma unroll
    for (int j = 0; j < QK_TOKENS; ++j) {
        const int t = t0 + j;
        const bool live = t < T;
        slot[j] = (write_kv && live) ? (long)__ldcg(slot_map + t) : -1;
        raw[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sizeof(TI) == 2 && live) raw[j] = ld_act4(src_base + (size_t)t * src_stride + (size_t)hh * 128 + lane * 4);
        if (rotate && live) {
            cs[j] = ld_act4(cos_t + (size_t)t * 64 + (lane & 15) * 4);
            sn[j] = ld_act4(sin_t + (size_t)t * 64 + (lane & 15) * 4);
        } else {
            cs[j] = make_float4(1.f, 1.f, 1.f, 1.f);
            sn[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (sizeof(TI) == 4) {
        // float32 partial products: three parts of all the tokens are requested at once and added in index order
        constexpr int PU = 3;
        for (int p0 = 0; p0 < nparts; p0 += PU) {
            float4 d[PU][QK_TOKENS];
#pragma unroll
            for (int pp = 0; pp < PU; ++pp)
#pragma unroll
                for (int j = 0; j < QK_TOKENS; ++j)
                    if (p0 + pp < nparts && t0 + j < T)
                        d[pp][j] = ld_act4(src_base + (size_t)(p0 + pp) * part_stride + (size_t)(t0 + j) * src_stride + (size_t)hh * 128 + lane * 4);
#pragma unroll
            for (int pp = 0; pp < PU; ++pp)
                if (p0 + pp < nparts) {
#pragma unroll
                    for (int j = 0; j < QK_TOKENS; ++j)
                        if (t0 + j < T) { raw[j].x += d[pp][j].x; raw[j].y += d[pp][j].y; raw[j].z += d[pp][j].z; raw[j].w += d[pp][j].w; }
                }
        }
    }
#pragma unroll
    for (int j = 0; j < QK_TOKENS; ++j) {
        const int t = t0 + j;
        float x0 = raw[j].x, x1 = raw[j].y, x2 = raw[j].z, x3 = raw[j].w;
        if (nw != nullptr) {
            const float ss = warp_sum(x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3);
            const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
            x0 = x0 * scale * wv.x; x1 = x1 * scale * wv.y; x2 = x2 * scale * wv.z; x3 = x3 * scale * wv.w;
        }
        if (cos_t != nullptr) {                                               // warp-uniform: v heads take part in the shuffles
            const float y0 = __shfl_xor_sync(0xffffffffu, x0, 16), y1 = __shfl_xor_sync(0xffffffffu, x1, 16);
            const float y2 = __shfl_xor_sync(0xffffffffu, x2, 16), y3 = __shfl_xor_sync(0xffffffffu, x3, 16);
            if (rotate) {
                if (lane < 16) {             // first half: a = own, b = partner: a c - b s
                    x0 = x0 * cs[j].x - y0 * sn[j].x; x1 = x1 * cs[j].y - y1 * sn[j].y; x2 = x2 * cs[j].z - y2 * sn[j].z; x3 = x3 * cs[j].w - y3 * sn[j].w;
                } else {                     // second half: a = partner, b = own: a s + b c
                    x0 = y0 * sn[j].x + x0 * cs[j].x; x1 = y1 * sn[j].y + x1 * cs[j].y; x2 = y2 * sn[j].z + x2 * cs[j].z; x3 = y3 * sn[j].w + x3 * cs[j].w;
                }
            }
        }
        if (t >= T || (!is_q && slot[j] < 0)) continue;                       // beyond the step, or a token without a cache slot
        __nv_bfloat162 o0 = __floats2bfloat162_rn(x0, x1), o1 = __floats2bfloat162_rn(x2, x3);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&o0); o.y = *reinterpret_cast<uint32_t*>(&o1);
        __nv_bfloat16* dst = is_q ? (q_out + (size_t)t * q_out_stride + (size_t)hh * 128)
                                  : ((is_k ? k_cache : v_cache) + ((size_t)slot[j] * nkv + hh) * 128);
        *reinterpret_cast<uint2*>(dst + lane * 4) = o;
    }
}

// One head row of the kernel below, held by 16 lanes with eight values each: norm, rotation, store.
// KIND 0 a query head, 1 a key head, 2 a value head (stored as it came): chosen per warp, so that
// nothing is decided per lane.
template <int KIND>
__device__ __forceinline__ void qk_pairs_row(const uint4 raw, bool live, int hh, int t, long slot, int l16, const float (&w)[8], bool normed,
                                             bool rotate, float eps, const float (&cs)[8], const float (&sn)[8],
                                             __nv_bfloat16* q_out, long q_out_stride, __nv_bfloat16* __restrict__ k_cache,
                                             __nv_bfloat16* __restrict__ v_cache, int nkv) {
    if (KIND == 2) {
        if (live && slot >= 0) *reinterpret_cast<uint4*>(v_cache + ((size_t)slot * nkv + hh) * 128 + l16 * 8) = raw;
        return;
    }
    float x[8];
    {
        const uint32_t w32[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w32[e]));
            x[2 * e] = f.x; x[2 * e + 1] = f.y;
        }
    }
    if (normed) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);        // over the 16 lanes of the row
        const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = x[e] * scale * w[e];
    }
    if (rotate) {
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = __shfl_xor_sync(0xffffffffu, x[e], 8);        // the rotation partner, 64 values away
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = fmaf(y[e], sn[e], x[e] * cs[e]);
    }
    if (!live || (KIND == 1 && slot < 0)) return;
    uint4 o;
    {
        __nv_bfloat162 p0b = __floats2bfloat162_rn(x[0], x[1]), p1b = __floats2bfloat162_rn(x[2], x[3]);
        __nv_bfloat162 p2b = __floats2bfloat162_rn(x[4], x[5]), p3b = __floats2bfloat162_rn(x[6], x[7]);
        o.x = *reinterpret_cast<uint32_t*>(&p0b); o.y = *reinterpret_cast<uint32_t*>(&p1b);
        o.z = *reinterpret_cast<uint32_t*>(&p2b); o.w = *reinterpret_cast<uint32_t*>(&p3b);
    }
    __nv_bfloat16* dst = KIND == 0 ? (q_out + (size_t)t * q_out_stride + (size_t)hh * 128) : (k_cache + ((size_t)slot * nkv + hh) * 128);
    *reinterpret_cast<uint4*>(dst + l16 * 8) = o;
}

// The same for many tokens with two head rows per warp: lanes 0-15 hold one row (eight values each,
// one 16-byte load), lanes 16-31 another; the sum of squares runs over 16 lanes, the rotation
// partner of a value is in lane ^ 8.  A CTA of eight warps takes four tokens, two warps each (the
// even and the odd pairs of heads), so a warp reads its token's rotation table once; HB pairs of
// rows are requested before the first is used.  A third of the instructions per row of the kernel
// above, which is what bounds it.
template <int HB>
__global__ void __launch_bounds__(256, 3)
qk_norm_rope_kv_write_hd128_pairs_kernel(
    const __nv_bfloat16* q, long q_stride, int nq, const __nv_bfloat16* __restrict__ k, long k_stride,
    const __nv_bfloat16* __restrict__ v, long v_stride, int nkv, __nv_bfloat16* q_out, long q_out_stride,
    const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int wdt, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int T) {
    griddep_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = lane >> 4, l16 = lane & 15;
    const int t = blockIdx.x * 4 + (warp & 3);
    const bool write_kv = (k != nullptr);
    const int n_heads = nq + (write_kv ? 2 * nkv : 0);
    float wq[8], wk[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) wq[e] = wk[e] = 1.f;
    if (q_norm_w != nullptr) {
        const float4 a = load4_dyn(q_norm_w, wdt, l16 * 8), b = load4_dyn(q_norm_w, wdt, l16 * 8 + 4);
        wq[0] = a.x; wq[1] = a.y; wq[2] = a.z; wq[3] = a.w; wq[4] = b.x; wq[5] = b.y; wq[6] = b.z; wq[7] = b.w;
    }
    if (k_norm_w != nullptr) {
        const float4 a = load4_dyn(k_norm_w, wdt, l16 * 8), b = load4_dyn(k_norm_w, wdt, l16 * 8 + 4);
        wk[0] = a.x; wk[1] = a.y; wk[2] = a.z; wk[3] = a.w; wk[4] = b.x; wk[5] = b.y; wk[6] = b.z; wk[7] = b.w;
    }
    griddep_wait();
    const bool live = t < T;
    const long slot = (write_kv && live) ? (long)__ldcg(slot_map + t) : -1;
    float cs[8], sn[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { cs[e] = 1.f; sn[e] = 0.f; }
    if (cos_t != nullptr && live) {
        const float* cp = cos_t + (size_t)t * 64 + (l16 & 7) * 8;
        const float* sp = sin_t + (size_t)t * 64 + (l16 & 7) * 8;
        const float4 c0 = ld_act4(cp), c1 = ld_act4(cp + 4), s0 = ld_act4(sp), s1 = ld_act4(sp + 4);
        cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    // the first half of a row is a c - b s, the second a s + b c with a, b = (own, partner) and (partner, own):
    // either way own * c + partner * (-+ s), so the sign goes into the sine once
    if (l16 < 8) {
#pragma unroll
        for (int e = 0; e < 8; ++e) sn[e] = -sn[e];
    }
    // this lane's heads: 2 * pair + half, pair = (warp >> 2) + 2 * gridDim.y * i + 2 * blockIdx.y
    const int pstep = 2 * gridDim.y;
    // with even numbers of query and of key/value heads the two rows of a pair are of one kind, which the warp
    // then decides once for all its lanes
    const bool pairs_of_a_kind = ((nq | nkv) & 1) == 0 || !write_kv && (nq & 1) == 0;
    const bool rot = cos_t != nullptr;
    for (int p0 = (warp >> 2) + 2 * blockIdx.y; pairs_of_a_kind && 2 * p0 < n_heads; p0 += pstep * HB) {
        uint4 raw[HB];
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            const int h0 = 2 * (p0 + pstep * u), head = h0 + half;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (live && h0 < n_heads) {
                const __nv_bfloat16* src = h0 < nq ? q + (size_t)t * q_stride + (size_t)head * 128
                                         : (h0 < nq + nkv ? k + (size_t)t * k_stride + (size_t)(head - nq) * 128
                                                          : v + (size_t)t * v_stride + (size_t)(head - nq - nkv) * 128);
                raw[u] = __ldcg(reinterpret_cast<const uint4*>(src + l16 * 8));
            }
        }
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            const int h0 = 2 * (p0 + pstep * u), head = h0 + half;
            if (h0 >= n_heads) break;
            if (h0 < nq)
                qk_pairs_row<0>(raw[u], live, head, t, slot, l16, wq, q_norm_w != nullptr, rot, eps, cs, sn, q_out, q_out_stride, k_cache, v_cache, nkv);
            else if (h0 < nq + nkv)
                qk_pairs_row<1>(raw[u], live, head - nq, t, slot, l16, wk, k_norm_w != nullptr, rot, eps, cs, sn, q_out, q_out_stride, k_cache, v_cache, nkv);
            else
                qk_pairs_row<2>(raw[u], live, head - nq - nkv, t, slot, l16, wk, false, false, eps, cs, sn, q_out, q_out_stride, k_cache, v_cache, nkv);
        }
    }
    for (int p0 = (warp >> 2) + 2 * blockIdx.y; !pairs_of_a_kind && 2 * p0 < n_heads; p0 += pstep * HB) {
        uint4 raw[HB];
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            const int head = 2 * (p0 + pstep * u) + half;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (live && head < n_heads) {
                const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
                const int hh = is_q ? head : (is_k ? head - nq : head - nq - nkv);
                const __nv_bfloat16* src = (is_q ? q : (is_k ? k : v)) + (size_t)t * (is_q ? q_stride : (is_k ? k_stride : v_stride)) + (size_t)hh * 128 + l16 * 8;
                raw[u] = __ldcg(reinterpret_cast<const uint4*>(src));
            }
        }
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            if (2 * (p0 + pstep * u) >= n_heads) break;                          // warp-uniform: both rows of the pair are beyond the heads
            const int head = 2 * (p0 + pstep * u) + half;
            const bool valid = live && head < n_heads;
            const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
            const int hh = is_q ? head : (is_k ? head - nq : head - nq - nkv);
            const bool normed = is_q ? (q_norm_w != nullptr) : (is_k && k_norm_w != nullptr);
            const bool rotate = cos_t != nullptr && (is_q || is_k);
            float x[8];
            {
                const uint32_t w32[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w32[e]));
                    x[2 * e] = f.x; x[2 * e + 1] = f.y;
                }
            }
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);        // over the 16 lanes of the row
            if (normed) {
                const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = x[e] * scale * (is_q ? wq[e] : wk[e]);
            }
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = __shfl_xor_sync(0xffffffffu, x[e], 8);        // the rotation partner, 64 values away
            if (rotate) {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = fmaf(y[e], sn[e], x[e] * cs[e]);
            }
            if (!valid || (!is_q && slot < 0)) continue;
            uint4 o;
            {
                __nv_bfloat162 p0b = __floats2bfloat162_rn(x[0], x[1]), p1b = __floats2bfloat162_rn(x[2], x[3]);
                __nv_bfloat162 p2b = __floats2bfloat162_rn(x[4], x[5]), p3b = __floats2bfloat162_rn(x[6], x[7]);
                o.x = *reinterpret_cast<uint32_t*>(&p0b); o.y = *reinterpret_cast<uint32_t*>(&p1b);
                o.z = *reinterpret_cast<uint32_t*>(&p2b); o.w = *reinterpret_cast<uint32_t*>(&p3b);
            }
            __nv_bfloat16* dst = is_q ? (q_out + (size_t)t * q_out_stride + (size_t)hh * 128)
                                      : ((is_k ? k_cache : v_cache) + ((size_t)slot * nkv + hh) * 128);
            *reinterpret_cast<uint4*>(dst + l16 * 8) = o;
        }
    }
}

// The same for many tokens (a prompt portion): a CTA of eight warps takes QK_TOKENS tokens and their
// heads (all of them, or every gridDim.y-th group of eight), warp w the heads w, w + 8, ...; the
// rotation table of the tokens is read once per warp, and the rows of HB heads x QK_TOKENS tokens
// are requested before the first is used.
template <int HB>
__global__ void __launch_bounds__(256)
qk_norm_rope_kv_write_hd128_rows_kernel(
    const __nv_bfloat16* q, long q_stride, int nq, const __nv_bfloat16* __restrict__ k, long k_stride,
    const __nv_bfloat16* __restrict__ v, long v_stride, int nkv, __nv_bfloat16* q_out, long q_out_stride,
    const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int wdt, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int T) {
    griddep_launch();
    const int t0 = blockIdx.x * QK_TOKENS, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool write_kv = (k != nullptr);
    const int n_heads = nq + (write_kv ? 2 * nkv : 0);
    float4 wq = make_float4(1.f, 1.f, 1.f, 1.f), wk = wq;
    if (q_norm_w != nullptr) wq = load4_dyn(q_norm_w, wdt, lane * 4);
    if (k_norm_w != nullptr) wk = load4_dyn(k_norm_w, wdt, lane * 4);
    griddep_wait();
    long slot[QK_TOKENS];
    float4 cs[QK_TOKENS], sn[QK_TOKENS];
#pragma unroll
    for (int j = 0; j < QK_TOKENS; ++j) {
        const int t = t0 + j;
        const bool live = t < T;
        slot[j] = (write_kv && live) ? (long)__ldcg(slot_map + t) : -1;
        if (cos_t != nullptr && live) {
            cs[j] = ld_act4(cos_t + (size_t)t * 64 + (lane & 15) * 4);
            sn[j] = ld_act4(sin_t + (size_t)t * 64 + (lane & 15) * 4);
        } else {
            cs[j] = make_float4(1.f, 1.f, 1.f, 1.f);
            sn[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    // heads of this warp: warp + 8 * (blockIdx.y + gridDim.y * i), i = 0, 1, ...; HB of them at a time
    const int hstep = 8 * gridDim.y;
    for (int h0 = warp + 8 * blockIdx.y; h0 < n_heads; h0 += hstep * HB) {
        float4 raw[HB][QK_TOKENS];
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            const int head = h0 + hstep * u;
            if (head < n_heads) {
                const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
                const int hh = is_q ? head : (is_k ? head - nq : head - nq - nkv);
                const __nv_bfloat16* src = (is_q ? q : (is_k ? k : v)) + (size_t)hh * 128 + lane * 4;
                const long stride = is_q ? q_stride : (is_k ? k_stride : v_stride);
#pragma unroll
                for (int j = 0; j < QK_TOKENS; ++j)
                    raw[u][j] = (t0 + j < T) ? ld_act4(src + (size_t)(t0 + j) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            const int head = h0 + hstep * u;
            if (head >= n_heads) break;
            const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
            const int hh = is_q ? head : (is_k ? head - nq : head - nq - nkv);
            const bool normed = is_q ? (q_norm_w != nullptr) : (is_k && k_norm_w != nullptr);
            const float4 wv = is_q ? wq : wk;
            const bool rotate = cos_t != nullptr && (is_q || is_k);
#pragma unroll
            for (int j = 0; j < QK_TOKENS; ++j) {
                const int t = t0 + j;
                float x0 = raw[u][j].x, x1 = raw[u][j].y, x2 = raw[u][j].z, x3 = raw[u][j].w;
                if (normed) {
                    const float ss = warp_sum(x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3);
                    const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
                    x0 = x0 * scale * wv.x; x1 = x1 * scale * wv.y; x2 = x2 * scale * wv.z; x3 = x3 * scale * wv.w;
                }
                if (rotate) {                                                      // the whole warp works on one head
                    const float y0 = __shfl_xor_sync(0xffffffffu, x0, 16), y1 = __shfl_xor_sync(0xffffffffu, x1, 16);
                    const float y2 = __shfl_xor_sync(0xffffffffu, x2, 16), y3 = __shfl_xor_sync(0xffffffffu, x3, 16);
                    if (lane < 16) {
                        x0 = x0 * cs[j].x - y0 * sn[j].x; x1 = x1 * cs[j].y - y1 * sn[j].y; x2 = x2 * cs[j].z - y2 * sn[j].z; x3 = x3 * cs[j].w - y3 * sn[j].w;
                    } else {
                        x0 = y0 * sn[j].x + x0 * cs[j].x; x1 = y1 * sn[j].y + x1 * cs[j].y; x2 = y2 * sn[j].z + x2 * cs[j].z; x3 = y3 * sn[j].w + x3 * cs[j].w;
                    }
                }
                if (t >= T || (!is_q && slot[j] < 0)) continue;
                __nv_bfloat162 o0 = __floats2bfloat162_rn(x0, x1), o1 = __floats2bfloat162_rn(x2, x3);
                uint2 o;
                o.x = *reinterpret_cast<uint32_t*>(&o0); o.y = *reinterpret_cast<uint32_t*>(&o1);
                __nv_bfloat16* dst = is_q ? (q_out + (size_t)t * q_out_stride + (size_t)hh * 128)
                                          : ((is_k ? k_cache : v_cache) + ((size_t)slot[j] * nkv + hh) * 128);
                *reinterpret_cast<uint2*>(dst + lane * 4) = o;
            }
        }
    }
}

// ---------------------------------------------------------------- dtype conversion (load time)
template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < n; idx += stride) out[idx] = from_f<TO>(to_f(in[idx]));
}

static inline int row_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

}  // namespace aien

using namespace aien;

AIEN_API int aien_embed_gather(const void* table, int table_dt, const int* ids, float* x,
                               int T, int H, int V, cudaStream_t stream) {
    if (T <= 0) return 0;
    AIEN_DISPATCH_DTYPE(table_dt, TW, (embed_gather_kernel<TW><<<T, row_threads(H), 0, stream>>>(
        (const TW*)table, ids, x, H, V)));
    return launch_status();
}

template <typename TD, typename TO>
static void launch_add_rmsnorm(float* x, const TD* delta, int nparts, size_t part_stride, const void* w, int w_dt,
                               float eps, TO* h, int T, int H, cudaStream_t stream) {
    const bool vec = (H % 4 == 0) && (((uintptr_t)x & 15) == 0) && (((uintptr_t)delta & 15) == 0) && (((uintptr_t)h & 15) == 0) &&
                     (((uintptr_t)w & 15) == 0) && (part_stride % 4 == 0);
#define VEC_CASE(NV, BS)                                                                                                          \
    do {                                                                                                                          \
        if (delta != nullptr && nparts > 1)                                                                                       \
            launch_chain(add_rmsnorm_vec_kernel<TD, TO, NV, true, BS>, dim3(T), dim3(BS), 0, stream, x, delta, nparts, part_stride, w, w_dt, eps, h, H); \
        else                                                                                                                      \
            launch_chain(add_rmsnorm_vec_kernel<TD, TO, NV, false, BS>, dim3(T), dim3(BS), 0, stream, x, delta, nparts, part_stride, w, w_dt, eps, h, H); \
    } while (0)
    // fewer rows than SMs: the rows' latency is the kernel's time, so more threads share a row
    const bool few_rows = T <= 148 && H > 256 * 4;
    if (vec && few_rows && H <= 1024 * 4)
        VEC_CASE(1, 1024);
    else if (vec && few_rows && H <= 1024 * 4 * 2)
        VEC_CASE(2, 1024);
    else if (vec && H <= 256 * 4 * 2)
        VEC_CASE(2, 256);
    else if (vec && H <= 256 * 4 * 4)
        VEC_CASE(4, 256);
    else if (vec && H <= 256 * 4 * 8)
        VEC_CASE(8, 256);
    else
        launch_chain(add_rmsnorm_kernel<TD, TO>, dim3(T), dim3(row_threads(H)), 0, stream, x, delta, nparts, part_stride, w, w_dt, eps, h, H);
#undef VEC_CASE
}

// delta: [nparts][T][H] (nparts >= 1; part_stride in elements) or null
AIEN_API int aien_add_rmsnorm(float* x, const void* delta, int delta_dt, int nparts, size_t part_stride,
                              const void* w, int w_dt, float eps, void* h, int h_dt, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (delta != nullptr && nparts < 1) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(delta_dt, TD, AIEN_DISPATCH_DTYPE(h_dt, TO,
        (launch_add_rmsnorm<TD, TO>(x, (const TD*)delta, nparts, part_stride, w, w_dt, eps, (TO*)h, T, H, stream))));
    return launch_status();
}

// out[t][i] = bfloat16(xw[t][i] * r_t), r_t = 1 / sqrt(sum_p ssq[p][t] / H + eps): finishes a norm
// whose weight is already inside xw and whose sums of squares came in per-CTA parts (see
// gemv_stream.cu), for a consumer that wants the normalised rows themselves.  T <= 16.
__global__ void __launch_bounds__(256)
scale_rows_ssq_kernel(const __nv_bfloat16* __restrict__ xw, long ld, const float* __restrict__ ssq, int parts, float eps,
                      __nv_bfloat16* __restrict__ out, long ldo, int H) {
    __shared__ float s_r;
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    if (threadIdx.x < 32) {
        float sq = 0.f;
        for (int p = threadIdx.x >> 4; p < parts; p += 2) sq += (threadIdx.x & 15) == 0 ? __ldcg(ssq + (size_t)p * 16 + t) : 0.f;
        sq += __shfl_xor_sync(0xffffffffu, sq, 16);
        if (threadIdx.x == 0) s_r = 1.0f / sqrtf(sq / (float)H + eps);
    }
    __syncthreads();
    const float r = s_r;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t)t * ldo + i] = __float2bfloat16_rn(ld_act(xw + (size_t)t * ld + i) * r);
}

AIEN_API int aien_scale_rows_ssq(const void* xw, long ld, const float* ssq, int parts, float eps, void* out, long ldo,
                                 int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (T > 16 || parts <= 0 || H <= 0) return AIEN_E_SHAPE;
    launch_chain(scale_rows_ssq_kernel, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)xw, ld, ssq, parts, eps,
                 (__nv_bfloat16*)out, ldo, H);
    return launch_status();
}

// token_ids[i] = prev[src[i]] where src[i] >= 0: a step whose tokens were sampled by the step before
// and have not been to the host takes them on the device.
__global__ void feed_token_ids_kernel(int* __restrict__ token_ids, const int* __restrict__ src, const int* __restrict__ prev, int T) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < T && src[i] >= 0) token_ids[i] = prev[src[i]];
}

AIEN_API int aien_feed_token_ids(int* token_ids, const int* src, const int* prev, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    feed_token_ids_kernel<<<(T + 127) / 128, 128, 0, stream>>>(token_ids, src, prev, T);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Cache housekeeping: the copy of a page (or of a state slot) in every run of a cache group, and zero fill.
// buf holds `slots` runs, slot_stride bytes apart; in each, n bytes at src_off are copied to dst_off
// (the two spans must not overlap).  16 bytes a thread where everything is 16-byte aligned.
__global__ void __launch_bounds__(256) copy_spans_kernel(uint8_t* __restrict__ buf, size_t slot_stride, size_t src_off, size_t dst_off, size_t n, int vec) {
    uint8_t* base = buf + (size_t)blockIdx.y * slot_stride;
    const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, step = (size_t)gridDim.x * blockDim.x;
    if (vec) {
        const uint4* s = reinterpret_cast<const uint4*>(base + src_off);
        uint4* d = reinterpret_cast<uint4*>(base + dst_off);
        for (size_t i = i0; i < n / 16; i += step) d[i] = s[i];
    } else {
        for (size_t i = i0; i < n; i += step) base[dst_off + i] = base[src_off + i];
    }
}

AIEN_API int aien_copy_spans(void* buf, size_t slot_stride, int slots, size_t src_off, size_t dst_off, size_t n, cudaStream_t stream) {
    if (slots <= 0 || n == 0) return 0;
    if (slots > 65535) return AIEN_E_SHAPE;
    if ((src_off < dst_off ? dst_off - src_off : src_off - dst_off) < n) return AIEN_E_SHAPE;        // overlapping spans
    const int vec = (((uintptr_t)buf | slot_stride | src_off | dst_off | n) & 15) == 0;
    const size_t items = vec ? n / 16 : n;
    const unsigned blocks = (unsigned)((items + 255) / 256 < 1024 ? (items + 255) / 256 : 1024);
    copy_spans_kernel<<<dim3(blocks, (unsigned)slots), 256, 0, stream>>>((uint8_t*)buf, slot_stride, src_off, dst_off, n, vec);
    return launch_status();
}

__global__ void __launch_bounds__(256) zero_fill_kernel(uint8_t* __restrict__ buf, size_t n, size_t head, size_t body16) {
    // head bytes up to the first 16-byte boundary, body16 vectors, then the tail
    const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, step = (size_t)gridDim.x * blockDim.x;
    uint4* body = reinterpret_cast<uint4*>(buf + head);
    for (size_t i = i0; i < body16; i += step) body[i] = make_uint4(0u, 0u, 0u, 0u);
    for (size_t i = i0; i < head; i += step) buf[i] = 0;
    for (size_t i = head + body16 * 16 + i0; i < n; i += step) buf[i] = 0;
}

AIEN_API int aien_zero_fill(void* buf, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    size_t head = (16 - ((uintptr_t)buf & 15)) & 15;
    if (head > n) head = n;
    const size_t body16 = (n - head) / 16;
    const size_t items = body16 > 256 ? body16 : 256;
    const unsigned blocks = (unsigned)((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
    zero_fill_kernel<<<blocks, 256, 0, stream>>>((uint8_t*)buf, n, head, body16);
    return launch_status();
}

AIEN_API int aien_gather_add_rows(const float* x, const void* delta, int delta_dt, int nparts, size_t part_stride,
                                  const int* rows, float* out, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    AIEN_DISPATCH_DTYPE(delta_dt, TD, (launch_chain(gather_add_rows_kernel<TD>, dim3(R), dim3(row_threads(H)), 0, stream,
        x, (const TD*)delta, nparts, part_stride, rows, out, H)));
    return launch_status();
}

AIEN_API int aien_add_residual(float* x, const void* delta, int delta_dt, int nparts, size_t part_stride, int T, int H,
                               cudaStream_t stream) {
    if (T <= 0 || H <= 0 || delta == nullptr) return 0;
    const size_t total = (size_t)T * H;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    AIEN_DISPATCH_DTYPE(delta_dt, TD, (launch_chain(add_residual_kernel<TD>, dim3(blocks), dim3(256), 0, stream,
        x, (const TD*)delta, nparts, part_stride, total)));
    return launch_status();
}

AIEN_API int aien_swiglu(const void* gu, void* out, int dt, int T, int I, int group, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (group < 0 || (group > 0 && I % group != 0)) return AIEN_E_SHAPE;
    const size_t total = (size_t)T * I;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    AIEN_DISPATCH_DTYPE(dt, TT, (launch_chain(swiglu_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (const TT*)gu, (TT*)out, I, group, total)));
    return launch_status();
}

AIEN_API int aien_rope_table(const int* positions, const double* inv_freq, float* cos_t, float* sin_t,
                             int T, int half, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    const int n = T * half;
    rope_table_kernel<<<(n + 127) / 128, 128, 0, stream>>>(positions, inv_freq, cos_t, sin_t, T, half);
    return launch_status();
}

// in_dt: dtype of q/k/v inputs ([nparts][T][...] when nparts > 1, float32 then); act_dt: dtype of q_out
AIEN_API int aien_qk_norm_rope_kv_write(
    const void* q, long q_stride, int nq, const void* k, long k_stride, const void* v, long v_stride, int nkv,
    int in_dt, int nparts, size_t part_stride, void* q_out, long q_out_stride,
    int hd, const void* q_norm_w, const void* k_norm_w, int w_dt, float eps,
    const float* cos_t, const float* sin_t, int rot, const int* slot_map,
    void* k_cache, void* v_cache, int act_dt, int kv_dt, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > AIEN_MAX_HEAD_DIM || rot < 0 || rot > hd || (rot & 1) || nparts < 1) return AIEN_E_SHAPE;
    if (T > 2147483647 / 1) return AIEN_E_SHAPE;
    const int n_heads = nq + (k != nullptr ? 2 * nkv : 0);
    dim3 grid(T, (n_heads + 3) / 4);
    if (grid.y > 65535) return AIEN_E_SHAPE;
    const bool a16 = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & (in_dt == AIEN_DT_F32 ? 15 : 7)) == 0 &&
                     (((uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 7) == 0 &&
                     ((q_stride | k_stride | v_stride | q_out_stride) & 3) == 0 && (part_stride & 3) == 0 &&
                     (((uintptr_t)q_norm_w | (uintptr_t)k_norm_w | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0;
    if (hd == 128 && act_dt == AIEN_DT_BF16 && (k == nullptr || kv_dt == AIEN_DT_BF16) && (cos_t == nullptr || rot == 128) && a16 &&
        ((in_dt == AIEN_DT_BF16 && nparts == 1) || in_dt == AIEN_DT_F32)) {
        const dim3 fast_grid((T + QK_TOKENS - 1) / QK_TOKENS, grid.y);
        // the heads of a token group are shared out over one, two or four CTAs: as many as make the fewest
        // waves of work over the GPU (three CTAs an SM), a CTA's fixed part (its tokens' rotation tables and
        // the norm weights) counted as 15 % of a whole token group
        unsigned head_ctas = 1;
        {
            int sms = 148, dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
            const long slots = 3L * sms;
            double best = 1e30;
            for (unsigned hc = 1; hc <= 4; hc *= 2) {
                if (hc > 1 && (int)(hc * 8) > n_heads) break;
                const double cost = (double)(((long)fast_grid.x * hc + slots - 1) / slots) * (1.0 / hc + 0.15);
                if (cost < best) { best = cost; head_ctas = hc; }
            }
        }
        const bool wide = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0 &&
                          ((q_stride | k_stride | v_stride | q_out_stride) & 7) == 0;
        if (in_dt == AIEN_DT_BF16 && T >= 128 && wide)
            launch_chain(qk_norm_rope_kv_write_hd128_pairs_kernel<3>, dim3(fast_grid.x, head_ctas), dim3(256), 0, stream,
                         (const __nv_bfloat16*)q, q_stride, nq, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, nkv,
                         (__nv_bfloat16*)q_out, q_out_stride, q_norm_w, k_norm_w, w_dt, eps, cos_t, sin_t, slot_map,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T);
        else if (in_dt == AIEN_DT_BF16 && T >= 128)
            launch_chain(qk_norm_rope_kv_write_hd128_rows_kernel<3>, dim3(fast_grid.x, head_ctas), dim3(256), 0, stream,
                         (const __nv_bfloat16*)q, q_stride, nq, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, nkv,
                         (__nv_bfloat16*)q_out, q_out_stride, q_norm_w, k_norm_w, w_dt, eps, cos_t, sin_t, slot_map,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T);
        else if (in_dt == AIEN_DT_BF16)
            launch_chain(qk_norm_rope_kv_write_hd128_kernel<__nv_bfloat16>, fast_grid, dim3(128), 0, stream,
                         (const __nv_bfloat16*)q, q_stride, nq, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, nkv,
                         nparts, part_stride, (__nv_bfloat16*)q_out, q_out_stride, q_norm_w, k_norm_w, w_dt, eps, cos_t, sin_t, slot_map,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T);
        else
            launch_chain(qk_norm_rope_kv_write_hd128_kernel<float>, fast_grid, dim3(128), 0, stream,
                         (const float*)q, q_stride, nq, (const float*)k, k_stride, (const float*)v, v_stride, nkv,
                         nparts, part_stride, (__nv_bfloat16*)q_out, q_out_stride, q_norm_w, k_norm_w, w_dt, eps, cos_t, sin_t, slot_map,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T);
        return launch_status();
    }
    AIEN_DISPATCH_DTYPE(in_dt, TI, AIEN_DISPATCH_DTYPE(act_dt, TC, AIEN_DISPATCH_DTYPE(kv_dt, TKV,
        (launch_chain(qk_norm_rope_kv_write_kernel<TI, TC, TKV>, grid, dim3(128), 0, stream,
            (const TI*)q, q_stride, nq, (const TI*)k, k_stride, (const TI*)v, v_stride, nkv, nparts, part_stride,
            (TC*)q_out, q_out_stride, hd, q_norm_w, k_norm_w, w_dt, eps, cos_t, sin_t, rot, slot_map,
            (TKV*)k_cache, (TKV*)v_cache)))));
    return launch_status();
}

AIEN_API int aien_convert(const void* in, int in_dt, void* out, int out_dt, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 32 ? (n + 255) / 256 : 148 * 32);
    AIEN_DISPATCH_DTYPE(in_dt, TI, AIEN_DISPATCH_DTYPE(out_dt, TO,
        (convert_kernel<TI, TO><<<blocks, 256, 0, stream>>>((const TI*)in, (TO*)out, n))));
    return launch_status();
}
