// Tile kernels that run on the CUDA cores: the memory-bound layer types (residual, pooling,
// layernorm, softmax, yolo, append) and the fp32-FFMA validation variant of the contraction tiles.
// Every function is executed by `nthr` cooperating threads of one CTA (thread ids 0..nthr-1) on
// one ninst tile.  Semantics follow the reference tile kernels, src/tiled_kernels.c (cited per
// function); activations are read with L1 bypass because other SMs produce them during the same
// kernel.
#pragma once
#include "device_types.h"
#include "../../include/aspen_b200.h"

// Barrier among the worker threads of a CTA only (the control warp does not take part).
__device__ __forceinline__ void worker_barrier(unsigned nthr) { asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory"); }

__device__ __forceinline__ float4 ldcg4(const float *p) { return __ldcg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float ldcg1(const float *p) { return __ldcg(p); }

// ref src/naive_kernels.c:11-57 (double-precision exp/tanh where the reference calls the double libm)
__device__ __forceinline__ float activate(float x, int act) {
    switch (act) {
        case RELU: return x > 0.f ? x : 0.f;
        case LEAKY_RELU: return x > 0.f ? x : (float)(0.1 * (double)x);
        case ELU: return x > 0.f ? x : (float)(0.1 * (exp((double)x) - 1.0));
        case SELU: return x > 0.f ? (float)(1.0507 * (double)x) : (float)(1.0507 * 1.67326 * (exp((double)x) - 1.0));
        case SIGMOID: return (float)(1.0 / (1.0 + exp(-(double)x)));
        case TANH: return (float)tanh((double)x);
        case GELU: return 0.5f * x * (1.f + erff(x * 0.7071067811865475f));
        case GELU_ACCURATE: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        default: return x;   // NO_ACTIVATION, LINEAR
    }
}

// GELU for the tensor-core epilogue, where 128 values per thread go through it.  The library erff / tanhf
// cost an order of magnitude more there than the contraction's own main loop; these forms are accurate to a
// few 1e-7 (far inside the TF32 bound) and branch-free.  The fp32 validation mode keeps `activate`.
//   erf: Abramowitz & Stegun 7.1.26, |error| <= 1.5e-7;  tanh(u) = 1 - 2 / (1 + exp(2u)), u clamped to +-15.
__device__ __forceinline__ float gelu_erf_fast(float x) {
    const float z = fabsf(x) * 0.7071067811865475f;
    const float t = __fdividef(1.f, fmaf(0.3275911f, z, 1.f));
    float p = fmaf(1.061405429f, t, -1.453152027f);
    p = fmaf(p, t, 1.421413741f);
    p = fmaf(p, t, -0.284496736f);
    p = fmaf(p, t, 0.254829592f);
    const float erf_abs = 1.f - p * t * __expf(-z * z);
    return 0.5f * x * (1.f + copysignf(erf_abs, x));
}
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    u = fminf(fmaxf(u, -15.f), 15.f);
    const float th = 1.f - __fdividef(2.f, 1.f + __expf(2.f * u));
    return 0.5f * x * (1.f + th);
}

// The tensor cores read only the upper 19 bits of an fp32 operand (TF32), i.e. they truncate.
// Truncation is biased toward zero and the bias compounds over a deep network, so every layer whose
// output feeds a tensor-core layer stores values already rounded to nearest TF32; the later
// truncation is then exact.  (Weights are rounded the same way when they are uploaded.)
__device__ __forceinline__ float tf32_round(float x) {
    unsigned u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}
__device__ __forceinline__ float finish(float x, const LayerDev &L) { x = activate(x, L.act); return L.round_out ? tf32_round(x) : x; }
__device__ __forceinline__ float store_round(float x, const LayerDev &L) { return L.round_out ? tf32_round(x) : x; }

// Output pixel (flattened column index) -> batch and top-left input coordinate of its window.
struct PixelWin { int b, ih0, iw0; };
__device__ __forceinline__ PixelWin pixel_window(const LayerDev &L, unsigned col) {
    unsigned hw = L.OH * L.OW;
    unsigned b = col / hw, r = col - b * hw;
    unsigned oh = r / L.OW, ow = r - oh * L.OW;
    PixelWin w;
    w.b = (int)b;
    w.ih0 = (int)(oh * L.stride) - (int)L.pad;
    w.iw0 = (int)(ow * L.stride) - (int)L.pad;
    return w;
}
// Pointer to the channel vector of input pixel (b, ih, iw), or nullptr when it is padding.
__device__ __forceinline__ const float *input_pixel(const LayerDev &L, const PixelWin &w, int kh, int kw) {
    int ih = w.ih0 + kh, iw = w.iw0 + kw;
    if (ih < 0 || ih >= (int)L.IH || iw < 0 || iw >= (int)L.IW) return nullptr;
    return L.in0 + ((size_t)(w.b * (int)L.IH + ih) * L.IW + iw) * L.ld0;
}

// ref src/tiled_kernels.c:613-638.  Pure streaming (12 bytes per element): four independent 16-byte
// load pairs are in flight per thread before the first use.
static __device__ __noinline__ void tile_residual(const LayerDev L, const TileDev T, unsigned tid, unsigned nthr) {
    const unsigned h4 = T.tile_h >> 2, tail = T.tile_h & 3;
    const unsigned total = T.tile_w * h4;
    constexpr int U = 4;
    for (unsigned i0 = tid; i0 < total; i0 += nthr * U) {
        float4 a[U], b[U];
        size_t off_o[U];
        #pragma unroll
        for (int u = 0; u < U; u++) {
            const unsigned i = i0 + u * nthr;
            if (i < total) {
                const unsigned n = i / h4, j = i - n * h4;
                const size_t col = T.pos_w + n;
                const unsigned m = T.pos_h + 4 * j;
                a[u] = ldcg4(L.in0 + col * L.ld0 + m);
                b[u] = ldcg4(L.in1 + col * L.ld1 + m);
                off_o[u] = col * L.ldc + m;
            }
        }
        #pragma unroll
        for (int u = 0; u < U; u++) {
            if (i0 + u * nthr < total) {
                float4 o = {finish(a[u].x + b[u].x, L), finish(a[u].y + b[u].y, L), finish(a[u].z + b[u].z, L), finish(a[u].w + b[u].w, L)};
                *reinterpret_cast<float4 *>(L.out + off_o[u]) = o;
            }
        }
    }
    if (tail) {
        for (unsigned i = tid; i < T.tile_w * tail; i += nthr) {
            const unsigned n = i / tail, m = T.pos_h + 4 * h4 + (i - n * tail);
            const size_t col = T.pos_w + n;
            L.out[col * L.ldc + m] = finish(ldcg1(L.in0 + col * L.ld0 + m) + ldcg1(L.in1 + col * L.ld1 + m), L);
        }
    }
}

// ref src/tiled_kernels.c:411-501.  Max ignores padded taps (all padded -> -inf); average divides by
// the full window size, padding counted.  A thread owns four channels of an output pixel and works on two such
// items at a time; the window's taps are fetched nine at a time (a whole 3 x 3 window), all loads of both items
// issued before the first is used (a tap outside the image reads nothing and contributes the neutral element),
// so the tile is bound by bandwidth instead of one load latency per tap.
template <bool IS_MAX>
static __device__ __noinline__ void tile_pool(const LayerDev L, const TileDev T, unsigned tid, unsigned nthr) {
    const unsigned h4 = T.tile_h >> 2, per_col = h4 + (T.tile_h & 3);
    const float inv = 1.f / (float)(L.KH * L.KW);
    const float init = IS_MAX ? -INFINITY : 0.f;
    const unsigned taps = L.KH * L.KW, total = T.tile_w * per_col;
    constexpr unsigned G = 9, U = 2;
    for (unsigned i0 = tid; i0 < total; i0 += nthr * U) {
        PixelWin w[U];
        unsigned m[U];
        size_t col[U];
        bool vec[U], live[U];
        float4 acc[U];
        #pragma unroll
        for (unsigned u = 0; u < U; u++) {
            const unsigned i = i0 + u * nthr;
            live[u] = i < total;
            const unsigned n = live[u] ? i / per_col : 0u, j = live[u] ? i - n * per_col : 0u;
            col[u] = T.pos_w + n;
            w[u] = pixel_window(L, (unsigned)col[u]);
            vec[u] = j < h4;
            m[u] = T.pos_h + (vec[u] ? 4 * j : 4 * h4 + (j - h4));
            acc[u] = make_float4(init, init, init, init);
        }
        unsigned kh = 0, kw = 0;
        for (unsigned t0 = 0; t0 < taps; t0 += G) {
            float4 v[U][G];
            #pragma unroll
            for (unsigned g = 0; g < G; g++) {
                const bool tap_ok = t0 + g < taps;
                #pragma unroll
                for (unsigned u = 0; u < U; u++) {
                    v[u][g] = make_float4(init, init, init, init);
                    if (tap_ok && live[u]) {
                        const float *src = input_pixel(L, w[u], (int)kh, (int)kw);
                        if (src) {
                            if (vec[u]) v[u][g] = ldcg4(src + m[u]);
                            else v[u][g].x = ldcg1(src + m[u]);
                        }
                    }
                }
                if (tap_ok && ++kw == L.KW) { kw = 0; kh++; }
            }
            #pragma unroll
            for (unsigned u = 0; u < U; u++) {
                #pragma unroll
                for (unsigned g = 0; g < G; g++) {
                    const float4 x = v[u][g];
                    if (IS_MAX) { acc[u].x = acc[u].x >= x.x ? acc[u].x : x.x; acc[u].y = acc[u].y >= x.y ? acc[u].y : x.y; acc[u].z = acc[u].z >= x.z ? acc[u].z : x.z; acc[u].w = acc[u].w >= x.w ? acc[u].w : x.w; }
                    else { acc[u].x += x.x; acc[u].y += x.y; acc[u].z += x.z; acc[u].w += x.w; }
                }
            }
        }
        #pragma unroll
        for (unsigned u = 0; u < U; u++) {
            if (!live[u]) continue;
            float4 a = acc[u];
            if (!IS_MAX) { a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv; }
            if (vec[u]) {
                float4 o = {finish(a.x, L), finish(a.y, L), finish(a.z, L), finish(a.w, L)};
                *reinterpret_cast<float4 *>(L.out + col[u] * L.ldc + m[u]) = o;
            } else {
                L.out[col[u] * L.ldc + m[u]] = finish(a.x, L);
            }
        }
    }
}

__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ref src/tiled_kernels.c:743-783: one pass mean / E[x^2], eps 1e-6, gain and shift.  One warp per column.
// A column of up to 1024 features is read ONCE: each lane keeps its up to eight 16-byte pieces in registers (all
// loads issued before the first use), the warp reduces sum and sum of squares, and the normalised values are
// written from the registers.  Longer or unaligned columns take the two-pass loop.
static __device__ __noinline__ void tile_layernorm(const LayerDev L, const TileDev T, unsigned tid, unsigned nthr) {
    const unsigned warp = tid >> 5, lane = tid & 31, nwarp = nthr >> 5;
    const unsigned M = T.tile_h;
    const float *gain = L.weight + T.pos_h;
    const float *shift = L.bias ? L.bias + T.pos_h : nullptr;
    const bool in_regs = M <= 1024u && (M & 3u) == 0u && ((L.ld0 | L.ldc | T.pos_h) & 3u) == 0u;
    for (unsigned n = warp; n < T.tile_w; n += nwarp) {
        const float *x = L.in0 + (size_t)(T.pos_w + n) * L.ld0 + T.pos_h;
        float *y = L.out + (size_t)(T.pos_w + n) * L.ldc + T.pos_h;
        if (in_regs) {
            float4 v[8];
            #pragma unroll
            for (unsigned q = 0; q < 8; q++) {
                const unsigned m = lane * 4u + q * 128u;
                v[q] = m < M ? ldcg4(x + m) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float s = 0.f, ss = 0.f;
            #pragma unroll
            for (unsigned q = 0; q < 8; q++) {
                s += v[q].x + v[q].y + v[q].z + v[q].w;
                ss += v[q].x * v[q].x + v[q].y * v[q].y + v[q].z * v[q].z + v[q].w * v[q].w;
            }
            s = warp_sum(s);
            ss = warp_sum(ss);
            const float mean = s / (float)M;
            const float var = ss / (float)M - mean * mean;
            const float inv = 1.f / sqrtf(var + 1e-6f);
            #pragma unroll
            for (unsigned q = 0; q < 8; q++) {
                const unsigned m = lane * 4u + q * 128u;
                if (m < M) {
                    const float4 g = *reinterpret_cast<const float4 *>(gain + m);
                    float4 o = {(v[q].x - mean) * inv * g.x, (v[q].y - mean) * inv * g.y, (v[q].z - mean) * inv * g.z, (v[q].w - mean) * inv * g.w};
                    if (shift) { const float4 b = *reinterpret_cast<const float4 *>(shift + m); o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w; }
                    o.x = store_round(o.x, L); o.y = store_round(o.y, L); o.z = store_round(o.z, L); o.w = store_round(o.w, L);
                    *reinterpret_cast<float4 *>(y + m) = o;
                }
            }
            continue;
        }
        float s = 0.f, ss = 0.f;
        const unsigned M4 = M & ~3u;
        for (unsigned m = lane * 4; m < M4; m += 128) {
            float4 v = ldcg4(x + m);
            s += v.x + v.y + v.z + v.w;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        for (unsigned m = M4 + lane; m < M; m += 32) { float v = ldcg1(x + m); s += v; ss += v * v; }
        s = warp_sum(s);
        ss = warp_sum(ss);
        float mean = s / (float)M;
        float var = ss / (float)M - mean * mean;
        float inv = 1.f / sqrtf(var + 1e-6f);
        for (unsigned m = lane * 4; m < M4; m += 128) {
            float4 v = ldcg4(x + m);
            float4 g = *reinterpret_cast<const float4 *>(gain + m);
            float4 o = {(v.x - mean) * inv * g.x, (v.y - mean) * inv * g.y, (v.z - mean) * inv * g.z, (v.w - mean) * inv * g.w};
            if (shift) { float4 b = *reinterpret_cast<const float4 *>(shift + m); o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w; }
            o.x = store_round(o.x, L); o.y = store_round(o.y, L); o.z = store_round(o.z, L); o.w = store_round(o.w, L);
            *reinterpret_cast<float4 *>(y + m) = o;
        }
        for (unsigned m = M4 + lane; m < M; m += 32) {
            float o = (ldcg1(x + m) - mean) * inv * gain[m];
            if (shift) o += shift[m];
            y[m] = store_round(o, L);
        }
    }
}

// ref src/tiled_kernels.c:640-673: max-subtracted softmax down each column.  One warp per column.
static __device__ __noinline__ void tile_softmax(const LayerDev L, const TileDev T, unsigned tid, unsigned nthr) {
    const unsigned warp = tid >> 5, lane = tid & 31, nwarp = nthr >> 5;
    const unsigned M = T.tile_h;
    for (unsigned n = warp; n < T.tile_w; n += nwarp) {
        const float *x = L.in0 + (size_t)(T.pos_w + n) * L.ld0 + T.pos_h;
        float *y = L.out + (size_t)(T.pos_w + n) * L.ldc + T.pos_h;
        float mx = -INFINITY;
        for (unsigned m = lane; m < M; m += 32) mx = fmaxf(mx, ldcg1(x + m));
        mx = warp_max(mx);
        float s = 0.f;
        for (unsigned m = lane; m < M; m += 32) s += expf(ldcg1(x + m) - mx);
        s = warp_sum(s);
        for (unsigned m = lane; m < M; m += 32) y[m] = store_round(expf(ldcg1(x + m) - mx) / s, L);
    }
}

// ref src/tiled_kernels.c:675-709: box decode of one detection head.
static __device__ __noinline__ void tile_yolo(const LayerDev L, const TileDev T, unsigned tid, unsigned nthr) {
    const unsigned C = L.p_out_c;
    const unsigned a_num = L.p_in_c / C, hw = L.IH * L.IW;
    for (unsigned i = tid; i < T.tile_w * C; i += nthr) {
        unsigned n = i / C, j = i - n * C;
        unsigned w_pos = T.pos_w + n;
        unsigned bidx = w_pos / (hw * a_num), b_num = w_pos % (hw * a_num);
        unsigned aidx = b_num / hw, wh = b_num % hw;
        unsigned hidx = wh / L.IW, widx = wh % L.IW;
        unsigned cidx = T.pos_h + aidx * C;
        const float *in = L.in0 + (size_t)(bidx * hw + hidx * L.IW + widx) * L.ld0 + cidx;
        float *out = L.out + (size_t)w_pos * L.ldc + T.pos_h;
        float v = ldcg1(in + j), o;
        if (j == 0) o = (1.0f / (1.0f + expf(-v)) + (float)widx) * (float)L.p_stride;
        else if (j == 1) o = (1.0f / (1.0f + expf(-v)) + (float)hidx) * (float)L.p_stride;
        else if (j == 2) o = expf(v) * L.anchors[2 * aidx];
        else if (j == 3) o = expf(v) * L.anchors[2 * aidx + 1];
        else o = 1.0f / (1.0f + expf(-v));
        out[j] = store_round(o, L);
    }
}

// ref src/tiled_kernels.c:711-741: nearest-neighbour upsample of PARENT_0 concatenated with PARENT_1.
static __device__ __noinline__ void tile_append(const LayerDev L, const TileDev T, unsigned tid, unsigned nthr) {
    const unsigned c1 = L.p_in_c, c2 = L.p_out_c - L.p_in_c, C = c1 + c2;
    const unsigned w2 = L.OW, w1 = L.IW, s = L.p_stride;
    for (unsigned i = tid; i < T.tile_w * C; i += nthr) {
        unsigned n = i / C, c = i - n * C;
        unsigned w_pos = T.pos_w + n;
        unsigned widx2 = w_pos % w2, hidx2 = w_pos / w2;
        unsigned widx1 = widx2 / s, hidx1 = hidx2 / s;
        float v = c < c1 ? ldcg1(L.in0 + (size_t)(hidx1 * w1 + widx1) * L.ld0 + c)
                         : ldcg1(L.in1 + (size_t)(hidx2 * w2 + widx2) * L.ld1 + (c - c1));
        L.out[(size_t)w_pos * L.ldc + c] = store_round(v, L);
    }
}

// ---- fp32 FFMA contraction tiles (validation mode) -----------------------------------------
// out[col n][row m] = epilogue( sum_k  W(m, k) * X(n, k) ), fp32 multiply-add in k order.
//   conv     ref src/tiled_kernels.c:161-297   X(n,k): input pixel taps (kh, kw, ic), zero padding
//   matmul   ref src/tiled_kernels.c:299-409   X(n,k): parent column n
//   connected ref src/tiled_kernels.c:502-612  X(n,k): flattened sample n
//   k-attn   ref src/tiled_kernels.c:784-932   W = keys, X = queries of one (batch, head); then
//                                              mask (-1e10), scale 1/sqrt(hd), exp, column normalise
//   v-attn   ref src/tiled_kernels.c:934-1038  W(m,k) = V[token k][feature m], X = probabilities
struct GemmView {
    const float *wbase;   // row m of W starts at wbase + m * wld (k contiguous) unless w_transposed
    size_t wld;
    bool w_transposed;    // v-attn: W(m,k) = wbase[k * wld + m]
    const float *xbase;   // non-conv: row n of X starts at xbase + n * xld
    size_t xld;
    unsigned K;
    bool conv;
};

__device__ __forceinline__ GemmView gemm_view(const LayerDev &L, const TileDev &T) {
    GemmView g;
    g.conv = false; g.w_transposed = false;
    switch (L.type) {
        case CONV_LAYER:
            g.wbase = L.weight + (size_t)T.pos_h * L.Kpad; g.wld = L.Kpad; g.xbase = L.in0; g.xld = L.ld0; g.K = L.K; g.conv = true;
            break;
        case MATMUL_LAYER:
            g.wbase = L.weight + (size_t)T.pos_h * L.Kpad; g.wld = L.Kpad; g.xbase = L.in0 + (size_t)T.pos_w * L.ld0; g.xld = L.ld0; g.K = L.K;
            break;
        case FC_LAYER:   // a convolution whose window is the whole input image (geometry set at upload)
            g.wbase = L.weight + (size_t)T.pos_h * L.Kpad; g.wld = L.Kpad; g.xbase = L.in0; g.xld = L.ld0; g.K = L.K; g.conv = true;
            break;
        case K_ATTENTION_LAYER: {
            unsigned b = T.pos_w / (L.seq * L.heads), head = (T.pos_w % (L.seq * L.heads)) / L.seq, q0 = T.pos_w % L.seq;
            g.wbase = L.in1 + (size_t)(b * L.seq + T.pos_h) * L.ld1 + head * L.hd; g.wld = L.ld1;
            g.xbase = L.in0 + (size_t)(b * L.seq + q0) * L.ld0 + head * L.hd; g.xld = L.ld0; g.K = L.hd;
            break;
        }
        default: {   // V_ATTENTION_LAYER
            unsigned b = T.pos_w / L.seq, head = T.pos_h / L.hd, q0 = T.pos_w % L.seq;
            g.wbase = L.in1 + (size_t)b * L.seq * L.ld1 + T.pos_h; g.wld = L.ld1; g.w_transposed = true;
            g.xbase = L.in0 + (size_t)((b * L.heads + head) * L.seq + q0) * L.ld0; g.xld = L.ld0; g.K = L.seq;
            break;
        }
    }
    return g;
}

// Layer-0 tile (service mode only): the uploaded input becomes the columns of the layer's activation matrix that the
// tile covers -- what the host-launched unpack / rounding / embedding-gather / padded-copy kernels do for a run that
// is launched per graph.  Sources are read through L2 (the host's DMA wrote them while this kernel was running).
static __device__ void tile_input(const InputDev &I, const LayerDev &L, const TileDev &T, unsigned tid, unsigned nthr) {
    const unsigned H = L.H;
    if (I.ids) {
        const unsigned m4 = T.tile_h >> 2;
        for (unsigned i = tid; i < T.tile_w * m4; i += nthr) {
            const unsigned c = i / m4, j = T.pos_h + (i - c * m4) * 4u;
            const size_t t = T.pos_w + c;
            int id = __ldcg(I.ids + t);
            id = id < 0 ? 0 : (id >= (int)I.emb_vocab ? (int)I.emb_vocab - 1 : id);
            float4 v = __ldg(reinterpret_cast<const float4 *>(I.emb_tok + (size_t)id * H + j));
            if (I.emb_pos) {
                const float4 p = __ldg(reinterpret_cast<const float4 *>(I.emb_pos + (size_t)(t % I.emb_seq) * H + j));
                v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
            }
            if (I.round) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
            *reinterpret_cast<float4 *>(L.out + t * L.ldc + j) = v;
        }
        return;
    }
    if (I.padded && I.stage && H <= 4u && T.pos_h == 0u) {
        // an image: one thread per pixel reads its (up to four) channels once and writes both copies
        const unsigned hw = I.IH * I.IW;
        for (unsigned c = tid; c < T.tile_w; c += nthr) {
            const unsigned w = T.pos_w + c, b = w / hw, r = w - b * hw, ih = r / I.IW, iw = r - ih * I.IW;
            const float *src = I.stage + (size_t)w * H;
            float *dst = L.out + (size_t)w * L.ldc;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            v.x = ldcg1(src);
            if (H > 1u) v.y = ldcg1(src + 1);
            if (H > 2u) v.z = ldcg1(src + 2);
            if (H > 3u) v.w = ldcg1(src + 3);
            if (I.round) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
            dst[0] = v.x;
            if (H > 1u) dst[1] = v.y;
            if (H > 2u) dst[2] = v.z;
            if (H > 3u) dst[3] = v.w;
            reinterpret_cast<float4 *>(I.padded)[((size_t)b * I.PH + ih + I.pad) * I.PW + iw + I.pad] = v;
        }
        return;
    }
    if ((I.stage || I.round) && ((T.tile_h | T.pos_h | L.ldc | H) & 3u) == 0u) {
        // 16-byte pieces: consecutive threads take consecutive pieces of a column
        const unsigned m4 = T.tile_h >> 2;
        for (unsigned i = tid; i < T.tile_w * m4; i += nthr) {
            const unsigned c = i / m4, m = T.pos_h + (i - c * m4) * 4u;
            const size_t w = T.pos_w + c;
            float *dst = L.out + w * L.ldc + m;
            float4 v = I.stage ? ldcg4(I.stage + w * H + m) : ldcg4(dst);
            if (I.round) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
            *reinterpret_cast<float4 *>(dst) = v;
        }
    } else if (I.stage || I.round)
        for (unsigned i = tid; i < T.tile_w * T.tile_h; i += nthr) {
            const unsigned c = i / T.tile_h, m = T.pos_h + (i - c * T.tile_h);
            const size_t w = T.pos_w + c;
            float *dst = L.out + w * L.ldc + m;
            float v = I.stage ? ldcg1(I.stage + w * H + m) : ldcg1(dst);
            *dst = I.round ? tf32_round(v) : v;
        }
    if (I.padded && T.pos_h == 0u)
        for (unsigned c = tid; c < T.tile_w; c += nthr) {
            const size_t w = T.pos_w + c, hw = (size_t)I.IH * I.IW, b = w / hw, r = w - b * hw;
            const unsigned ih = (unsigned)(r / I.IW), iw = (unsigned)(r - (size_t)ih * I.IW);
            const float *src = I.stage ? I.stage + w * H : L.out + w * L.ldc;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            v.x = ldcg1(src);
            if (I.IC > 1) v.y = ldcg1(src + 1);
            if (I.IC > 2) v.z = ldcg1(src + 2);
            if (I.IC > 3) v.w = ldcg1(src + 3);
            if (I.round) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
            reinterpret_cast<float4 *>(I.padded)[(b * I.PH + ih + I.pad) * I.PW + iw + I.pad] = v;
        }
}

static __device__ void tile_gemm_ffma(const LayerDev L, const TileDev T, unsigned tid, unsigned nthr) {
    const GemmView g = gemm_view(L, T);
    const unsigned mg = (T.tile_h + 3) >> 2;             // groups of 4 output rows
    const bool vec = !g.w_transposed && (g.conv ? (L.IC & 3) == 0 : (g.K & 3) == 0) && L.a_vec4;
    const bool is_k = L.type == K_ATTENTION_LAYER;
    const float scale = is_k ? sqrtf((float)L.hd) : 1.f;
    const unsigned q0 = is_k ? T.pos_w % L.seq : 0;
    for (unsigned i = tid; i < mg * T.tile_w; i += nthr) {
        const unsigned n = i % T.tile_w, m0 = (i / T.tile_w) * 4;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const float *w[4];
        for (int r = 0; r < 4; r++) {
            unsigned m = m0 + r < T.tile_h ? m0 + r : T.tile_h - 1;   // clamp: duplicates are discarded below
            w[r] = g.w_transposed ? g.wbase + m : g.wbase + (size_t)m * g.wld;
        }
        if (g.conv) {
            PixelWin pw = pixel_window(L, T.pos_w + n);
            unsigned k = 0;
            for (int kh = 0; kh < (int)L.KH; kh++)
                for (int kw = 0; kw < (int)L.KW; kw++, k += L.IC) {
                    const float *x = input_pixel(L, pw, kh, kw);
                    if (!x) continue;
                    if (vec) {
                        for (unsigned c = 0; c < L.IC; c += 4) {
                            float4 xv = ldcg4(x + c);
                            for (int r = 0; r < 4; r++) {
                                float4 wv = *reinterpret_cast<const float4 *>(w[r] + k + c);
                                acc[r] = fmaf(wv.x, xv.x, acc[r]); acc[r] = fmaf(wv.y, xv.y, acc[r]);
                                acc[r] = fmaf(wv.z, xv.z, acc[r]); acc[r] = fmaf(wv.w, xv.w, acc[r]);
                            }
                        }
                    } else {
                        for (unsigned c = 0; c < L.IC; c++) {
                            float xv = ldcg1(x + c);
                            for (int r = 0; r < 4; r++) acc[r] = fmaf(w[r][k + c], xv, acc[r]);
                        }
                    }
                }
        } else {
            const float *x = g.xbase + (size_t)n * g.xld;
            if (vec) {
                for (unsigned k = 0; k < g.K; k += 4) {
                    float4 xv = ldcg4(x + k);
                    for (int r = 0; r < 4; r++) {
                        float4 wv = ldcg4(w[r] + k);
                        acc[r] = fmaf(wv.x, xv.x, acc[r]); acc[r] = fmaf(wv.y, xv.y, acc[r]);
                        acc[r] = fmaf(wv.z, xv.z, acc[r]); acc[r] = fmaf(wv.w, xv.w, acc[r]);
                    }
                }
            } else {
                for (unsigned k = 0; k < g.K; k++) {
                    float xv = ldcg1(x + k);
                    for (int r = 0; r < 4; r++) acc[r] = fmaf(ldcg1(g.w_transposed ? w[r] + (size_t)k * g.wld : w[r] + k), xv, acc[r]);
                }
            }
        }
        float *o = L.out + (size_t)(T.pos_w + n) * L.ldc + T.pos_h + m0;
        for (int r = 0; r < 4; r++) {
            if (m0 + r >= T.tile_h) break;
            float v = acc[r];
            if (is_k) {
                if (L.masked && (T.pos_h + m0 + r) > (q0 + n)) v = -1e10f;
                v = expf(v / scale);
            } else if (L.type != V_ATTENTION_LAYER) {
                if (L.bias) v += L.bias[T.pos_h + m0 + r];
                v = activate(v, L.act);
            }
            o[r] = v;
        }
    }
    if (is_k) {   // normalise every column by its sum (no max subtraction, as the reference)
        worker_barrier(nthr);
        const unsigned warp = tid >> 5, lane = tid & 31, nwarp = nthr >> 5;
        for (unsigned n = warp; n < T.tile_w; n += nwarp) {
            float *o = L.out + (size_t)(T.pos_w + n) * L.ldc + T.pos_h;
            float s = 0.f;
            for (unsigned m = lane; m < T.tile_h; m += 32) s += ldcg1(o + m);
            s = warp_sum(s);
            for (unsigned m = lane; m < T.tile_h; m += 32) o[m] = ldcg1(o + m) / s;
        }
    }
}
