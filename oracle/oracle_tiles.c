/*
 * TEST INFRASTRUCTURE ONLY -- the CPU oracle.  Never linked into, imported by or called from the
 * product library; only tests/, the smoke check and the benchmark's cpu_baseline leg use it.
 *
 * Plain-C restatement of the arithmetic of the reference's tile kernels, one whole layer at a
 * time.  Tile VALUES do not depend on how a layer is cut into ninst tiles, so a layer-level
 * function is an exact statement of what every tile of that layer must contain.
 *
 * Data layout is the reference's: an activation matrix is column-major, one column per pixel /
 * token (index b*OH*OW + oh*OW + ow, or b*S + s), the channels / features of a column contiguous
 * (ref include/nasm.h:33-37, src/apu_nasm.c:892-901).  Here columns are PACKED (stride == rows).
 * Weights are in weight-file order: conv OIHW, connected [O][C][H][W], matmul [M][K]
 * (ref src/apu_file_io.c:226-255).
 *
 * Parity pinned: tests/test_oracle.py checks these functions against fixtures produced by the
 * unmodified reference (tests/golden/make_golden.py) and, when oracle/_ref is built, against the
 * reference live on random shapes.
 */
#include <math.h>
#include <stddef.h>
#include <string.h>

enum { ACT_NONE = 0, ACT_SIGMOID = 1, ACT_LINEAR = 2, ACT_TANH = 3, ACT_RELU = 4, ACT_LEAKY = 5, ACT_ELU = 6, ACT_SELU = 7,
       ACT_GELU = 8, ACT_GELU_ACC = 9 };   /* LAYER_ACT values, ref include/aspen.h:64 */

/* ref src/naive_kernels.c:11-57 */
void oracle_activate(float *x, size_t n, int act)
{
    for (size_t i = 0; i < n; i++) {
        float v = x[i];
        switch (act) {
            case ACT_RELU: v = v > 0 ? v : 0; break;
            case ACT_LEAKY: v = v > 0 ? v : 0.1 * v; break;
            case ACT_ELU: v = v > 0 ? v : 0.1 * (exp(v) - 1); break;
            case ACT_SELU: v = v > 0 ? 1.0507 * v : 1.0507 * 1.67326 * (exp(v) - 1); break;
            case ACT_SIGMOID: v = 1 / (1 + exp(-v)); break;
            case ACT_TANH: v = tanh(v); break;
            case ACT_GELU: v = 0.5 * v * (1 + erff(v * 0.7071067811865475f)); break;
            case ACT_GELU_ACC: v = 0.5 * v * (1 + tanhf(0.7978845608028654f * (v + 0.044715 * v * v * v))); break;
            default: break;
        }
        x[i] = v;
    }
}

/* ref src/tiled_kernels.c:161-297 (+ prepare_input 3-45): out[pix][oc] = act(bias[oc] + sum over
 * (kh, kw, ic) of w[oc][ic][kh][kw] * in[b, oh*s+kh-p, ow*s+kw-p][ic]); out-of-image taps read zero.
 * The dilation parameter is parsed by the reference but not used by its tile kernel (line 25-26). */
void oracle_conv2d(const float *in, const float *w, const float *bias, float *out, int B, int IH, int IW, int IC, int OC,
                   int KH, int KW, int stride, int pad, int act)
{
    const int OH = (IH + 2 * pad - (KH - 1) - 1) / stride + 1, OW = (IW + 2 * pad - (KW - 1) - 1) / stride + 1;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int oh = 0; oh < OH; oh++)
            for (int ow = 0; ow < OW; ow++) {
                float *o = out + ((size_t)(b * OH + oh) * OW + ow) * OC;
                for (int oc = 0; oc < OC; oc++) {
                    float acc = 0;
                    for (int kh = 0; kh < KH; kh++) {
                        int ih = oh * stride + kh - pad;
                        if (ih < 0 || ih >= IH) continue;
                        for (int kw = 0; kw < KW; kw++) {
                            int iw = ow * stride + kw - pad;
                            if (iw < 0 || iw >= IW) continue;
                            const float *x = in + ((size_t)(b * IH + ih) * IW + iw) * IC;
                            const float *ww = w + (size_t)oc * IC * KH * KW + (size_t)kh * KW + kw;
                            for (int ic = 0; ic < IC; ic++) acc += ww[(size_t)ic * KH * KW] * x[ic];
                        }
                    }
                    o[oc] = acc + (bias ? bias[oc] : 0.f);
                }
                oracle_activate(o, OC, act);
            }
}

/* ref src/tiled_kernels.c:299-409: out[n][m] = act(bias[m] + sum_k w[m][k] * in[n][k]) */
void oracle_matmul(const float *in, const float *w, const float *bias, float *out, int N, int K, int M, int act)
{
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const float *x = in + (size_t)n * K;
        float *o = out + (size_t)n * M;
        for (int m = 0; m < M; m++) {
            const float *ww = w + (size_t)m * K;
            float acc = 0;
            for (int k = 0; k < K; k++) acc += ww[k] * x[k];
            o[m] = acc + (bias ? bias[m] : 0.f);
        }
        oracle_activate(o, M, act);
    }
}

/* ref src/tiled_kernels.c:502-612: the sample's NHWC activations flattened in (h, w, c) order against
 * weights given as [O][C][H][W] (the reference re-orders them to (h, w, c), src/apu.c:24-31). */
void oracle_fully_connected(const float *in, const float *w, const float *bias, float *out, int B, int IH, int IW, int IC,
                            int OC, int act)
{
    #pragma omp parallel for schedule(static)
    for (int b = 0; b < B; b++) {
        float *o = out + (size_t)b * OC;
        for (int oc = 0; oc < OC; oc++) {
            float acc = 0;
            for (int h = 0; h < IH; h++)
                for (int x = 0; x < IW; x++)
                    for (int c = 0; c < IC; c++)
                        acc += w[(((size_t)oc * IC + c) * IH + h) * IW + x] * in[(((size_t)b * IH + h) * IW + x) * IC + c];
            o[oc] = acc + (bias ? bias[oc] : 0.f);
        }
        oracle_activate(o, OC, act);
    }
}

/* ref src/tiled_kernels.c:411-455: maximum over the window's in-image taps; -inf if there is none. */
void oracle_maxpool2d(const float *in, float *out, int B, int IH, int IW, int C, int KH, int KW, int stride, int pad, int act)
{
    const int OH = (IH + 2 * pad - (KH - 1) - 1) / stride + 1, OW = (IW + 2 * pad - (KW - 1) - 1) / stride + 1;
    for (int b = 0; b < B; b++)
        for (int oh = 0; oh < OH; oh++)
            for (int ow = 0; ow < OW; ow++) {
                float *o = out + ((size_t)(b * OH + oh) * OW + ow) * C;
                for (int c = 0; c < C; c++) o[c] = -INFINITY;
                for (int kh = 0; kh < KH; kh++)
                    for (int kw = 0; kw < KW; kw++) {
                        int ih = oh * stride + kh - pad, iw = ow * stride + kw - pad;
                        if (ih < 0 || ih >= IH || iw < 0 || iw >= IW) continue;
                        const float *x = in + ((size_t)(b * IH + ih) * IW + iw) * C;
                        for (int c = 0; c < C; c++) o[c] = o[c] >= x[c] ? o[c] : x[c];
                    }
                oracle_activate(o, C, act);
            }
}

/* ref src/tiled_kernels.c:456-501: sum of the in-image taps divided by the FULL window size. */
void oracle_avgpool2d(const float *in, float *out, int B, int IH, int IW, int C, int KH, int KW, int stride, int pad, int act)
{
    const int OH = (IH + 2 * pad - (KH - 1) - 1) / stride + 1, OW = (IW + 2 * pad - (KW - 1) - 1) / stride + 1;
    for (int b = 0; b < B; b++)
        for (int oh = 0; oh < OH; oh++)
            for (int ow = 0; ow < OW; ow++) {
                float *o = out + ((size_t)(b * OH + oh) * OW + ow) * C;
                for (int c = 0; c < C; c++) o[c] = 0;
                for (int kh = 0; kh < KH; kh++)
                    for (int kw = 0; kw < KW; kw++) {
                        int ih = oh * stride + kh - pad, iw = ow * stride + kw - pad;
                        if (ih < 0 || ih >= IH || iw < 0 || iw >= IW) continue;
                        const float *x = in + ((size_t)(b * IH + ih) * IW + iw) * C;
                        for (int c = 0; c < C; c++) o[c] += x[c];
                    }
                for (int c = 0; c < C; c++) o[c] /= (float)(KH * KW);
                oracle_activate(o, C, act);
            }
}

/* ref src/tiled_kernels.c:613-638: activation AFTER the add. */
void oracle_residual(const float *a, const float *b, float *out, size_t n, int act)
{
    for (size_t i = 0; i < n; i++) out[i] = a[i] + b[i];
    oracle_activate(out, n, act);
}

/* ref src/tiled_kernels.c:743-783: single pass mean and E[x^2], variance E[x^2]-mean^2, eps 1e-6. */
void oracle_layernorm(const float *in, const float *gain, const float *shift, float *out, int N, int M)
{
    for (int n = 0; n < N; n++) {
        const float *x = in + (size_t)n * M;
        float *o = out + (size_t)n * M;
        float mean = 0, var = 0;
        for (int m = 0; m < M; m++) { mean += x[m]; var += x[m] * x[m]; }
        mean /= M;
        var /= M;
        var -= mean * mean;
        var = 1 / sqrtf(var + 1e-6f);
        for (int m = 0; m < M; m++) {
            o[m] = (x[m] - mean) * var * gain[m];
            if (shift) o[m] += shift[m];
        }
    }
}

/* ref src/tiled_kernels.c:640-673: max-subtracted softmax down each column. */
void oracle_softmax(const float *in, float *out, int N, int M)
{
    for (int n = 0; n < N; n++) {
        const float *x = in + (size_t)n * M;
        float *o = out + (size_t)n * M;
        float mx = x[0], sum = 0;
        for (int m = 1; m < M; m++) mx = mx >= x[m] ? mx : x[m];
        for (int m = 0; m < M; m++) { o[m] = expf(x[m] - mx); sum += o[m]; }
        for (int m = 0; m < M; m++) o[m] /= sum;
    }
}

/* ref src/tiled_kernels.c:784-932.  q, k: [B*S][hidden].  out: [(b*heads + head)*S + query][key]
 *   s = sum_d k[b, key, head*hd + d] * q[b, query, head*hd + d]
 *   masked and key > query  ->  s = -1e10   (before scaling)
 *   p = exp(s / sqrtf(hd));  p /= sum over keys        (no maximum subtraction) */
void oracle_k_attention(const float *q, const float *k, float *out, int B, int S, int heads, int hidden, int masked)
{
    const int hd = hidden / heads;
    const float scale = sqrtf((float)hd);
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int h = 0; h < heads; h++)
            for (int n = 0; n < S; n++) {
                float *o = out + ((size_t)(b * heads + h) * S + n) * S;
                const float *qq = q + (size_t)(b * S + n) * hidden + h * hd;
                float total = 0;
                for (int m = 0; m < S; m++) {
                    const float *kk = k + (size_t)(b * S + m) * hidden + h * hd;
                    float s = 0;
                    for (int d = 0; d < hd; d++) s += kk[d] * qq[d];
                    if (masked && m > n) s = -1e10f;
                    o[m] = expf(s / scale);
                    total += o[m];
                }
                for (int m = 0; m < S; m++) o[m] /= total;
            }
}

/* ref src/tiled_kernels.c:934-1038.  p: [(b*heads + head)*S + query][key], v: [B*S][hidden].
 *   out[b*S + query][head*hd + d] = sum over keys of v[b, key, head*hd + d] * p[(b, head, query)][key] */
void oracle_v_attention(const float *p, const float *v, float *out, int B, int S, int heads, int hidden)
{
    const int hd = hidden / heads;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int n = 0; n < S; n++)
            for (int m = 0; m < hidden; m++) {
                const int h = m / hd;
                const float *pp = p + ((size_t)(b * heads + h) * S + n) * S;
                float acc = 0;
                for (int s = 0; s < S; s++) acc += v[(size_t)(b * S + s) * hidden + m] * pp[s];
                out[(size_t)(b * S + n) * hidden + m] = acc;
            }
}

/* ref src/tiled_kernels.c:675-709: box decode of one detection head.  in: [B*IH*IW][a_num * C] (C = classes + 5),
 * out: [B * a_num * IH * IW][C], column b*(a_num*IH*IW) + a*(IH*IW) + h*IW + w.
 *   x = (sigmoid(in0) + w) * stride,  y = (sigmoid(in1) + h) * stride,
 *   bw = exp(in2) * anchor[2a],       bh = exp(in3) * anchor[2a+1],   the rest: sigmoid. */
void oracle_yolo(const float *in, const float *anchors, float *out, int B, int IH, int IW, int IC, int C, int stride)
{
    const int a_num = IC / C, hw = IH * IW;
    for (int b = 0; b < B; b++)
        for (int a = 0; a < a_num; a++)
            for (int h = 0; h < IH; h++)
                for (int w = 0; w < IW; w++) {
                    const float *x = in + ((size_t)(b * hw) + h * IW + w) * IC + a * C;
                    float *o = out + ((size_t)(b * a_num + a) * hw + h * IW + w) * C;
                    o[0] = (1.0f / (1.0f + expf(-x[0])) + w) * stride;
                    o[1] = (1.0f / (1.0f + expf(-x[1])) + h) * stride;
                    o[2] = expf(x[2]) * anchors[2 * a];
                    o[3] = expf(x[3]) * anchors[2 * a + 1];
                    for (int j = 4; j < C; j++) o[j] = 1.0f / (1.0f + expf(-x[j]));
                }
}

/* ref src/tiled_kernels.c:711-741: PARENT_0 ([B*IH*IW][C1]) upsampled by `stride` (nearest neighbour), then
 * PARENT_1's channels ([B*OH*OW][C2], OH = IH*stride) behind it: out [B*OH*OW][C1 + C2]. */
void oracle_append(const float *in1, const float *in2, float *out, int B, int IH, int IW, int C1, int C2, int stride)
{
    const int OH = IH * stride, OW = IW * stride;
    for (int b = 0; b < B; b++)
        for (int h = 0; h < OH; h++)
            for (int w = 0; w < OW; w++) {
                const size_t col = ((size_t)b * OH + h) * OW + w;
                float *o = out + col * (C1 + C2);
                memcpy(o, in1 + (((size_t)b * IH + h / stride) * IW + w / stride) * C1, (size_t)C1 * sizeof(float));
                memcpy(o + C1, in2 + col * C2, (size_t)C2 * sizeof(float));
            }
}
