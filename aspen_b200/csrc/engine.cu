// Host side of the device engine: uploads weights and flattened tile graphs, owns the stream,
// launches the persistent scheduler, and moves inputs / results.  The only translation unit of
// the library that calls the CUDA runtime.  There is no CPU execution path: without a usable
// sm_100 device every entry point fails with an error.
#include "internal.h"
#include "scheduler.cuh"

#include <cuda.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <mutex>
#include <sched.h>
#include <unordered_map>

#define CUDA_TRY(expr)                                                                          \
    do {                                                                                        \
        cudaError_t err__ = (expr);                                                             \
        if (err__ != cudaSuccess) {                                                             \
            ASPEN_ERR("CUDA error %s at %s: %s\n", cudaGetErrorName(err__), #expr, cudaGetErrorString(err__)); \
            return -1;                                                                          \
        }                                                                                       \
    } while (0)

struct Engine;
static int svc_halt(Engine *e);
static int svc_run(Engine *e, const std::vector<nasm_t *> &nasms);
static int svc_wait(nasm_t *nasm);
static int svc_attach(Engine *e, nasm_t *nasm, const void *input_host, const int *ids_host, bool keep_input);
static bool svc_done(const struct DeviceNasm *dn);

static thread_local int g_device = -1;

extern "C" int aspen_b200_set_device(int device) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) {
        ASPEN_ERR("aspen_b200_set_device: device %d not available (%d visible)\n", device, n);
        return -1;
    }
    g_device = device;
    return cudaSetDevice(device) == cudaSuccess ? 0 : -1;
}

// Whether every layer's output stays readable after a run (the default), or outputs that only feed a residual add
// fused into their producer are left unwritten (1 = keep all, 0 = drop those).  Read when a graph's device image is built.
static thread_local int g_keep_hidden = -1;

extern "C" void aspen_b200_set_hidden_states(int keep) { g_keep_hidden = keep ? 1 : 0; }

static bool keep_hidden_states() {
    if (g_keep_hidden >= 0) return g_keep_hidden != 0;
    const char *v = getenv("ASPEN_B200_HIDDEN_STATES");
    return !(v && *v && atoi(v) == 0);
}

int engine_current_device() {
    if (g_device >= 0) return g_device;
    if (const char *v = getenv("ASPEN_B200_DEVICE")) {     // for callers that cannot call aspen_b200_set_device
        int n = 0, want = atoi(v);
        if (*v && cudaGetDeviceCount(&n) == cudaSuccess && want >= 0 && want < n) return want;
    }
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) return 0;
    return d;
}

// ---- device copies of a dnn's weights ----------------------------------------------------------
struct DeviceDnn {
    int device = 0;
    // per layer, per precision mode (0: rounded to TF32, 1: exact fp32)
    std::vector<float *> weight[2];
    std::vector<float *> bias;
    std::vector<float *> anchors;
    std::vector<unsigned> kpad;
    std::vector<float *> weight_rows;   // tensor-core path, input convolutions with <= 4 channels: k = (kh, [kw][4] padded to 32)
    std::vector<unsigned> ic_pad;     // conv on the network input with IC % 4 != 0: channels padded to this many (0: not padded)
    bool have[2] = {false, false};
    float *emb_token = nullptr, *emb_position = nullptr;   // embedding tables, uploaded on first use
};

static float round_to_tf32(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x00001000u;          // round to nearest, ties away: 13 mantissa bits are dropped
    u &= 0xffffe000u;
    memcpy(&x, &u, 4);
    return x;
}

static int upload_weights(aspen_dnn_t *dnn, int device, int precision, DeviceDnn **out) {
    if (device < 0 || device >= 16) { ASPEN_ERR("device index %d out of range\n", device); return -1; }
    DeviceDnn *dd = dnn->dev[device];
    if (!dd) {
        dd = new DeviceDnn();
        dd->device = device;
        dd->weight[0].assign(dnn->num_layers, nullptr);
        dd->weight[1].assign(dnn->num_layers, nullptr);
        dd->bias.assign(dnn->num_layers, nullptr);
        dd->anchors.assign(dnn->num_layers, nullptr);
        dd->kpad.assign(dnn->num_layers, 0);
        dd->ic_pad.assign(dnn->num_layers, 0);
        dd->weight_rows.assign(dnn->num_layers, nullptr);
        dnn->dev[device] = dd;
    }
    *out = dd;
    if (dd->have[precision]) return 0;
    for (unsigned i = 0; i < dnn->num_layers; i++) {
        aspen_layer_t &l = dnn->layers[i];
        aspen_tensor_t *w = l.tensors[WEIGHT_TENSOR], *b = l.tensors[BIAS_TENSOR], *a = l.tensors[ANCHOR_TENSOR];
        if (w) {
            unsigned rows = layer_weight_rows(&l);
            unsigned k = l.type == LAYERNORM_LAYER ? 1 : layer_contraction_k(&l);
            // A convolution straight on the network input with an odd channel count (the 3-channel
            // stem): the input matrix keeps its pad rows zero, so the device copy pads every tap to a
            // multiple of 4 channels with zero weights and the tile reads 16-byte pieces.
            unsigned ic = l.params[IN_C], icp = ic;
            if (l.type == CONV_LAYER && l.parent_layers[PARENT_0] && l.parent_layers[PARENT_0]->type == INPUT_LAYER && ic % 4 != 0) {
                icp = (unsigned)round_up(ic, 4);
                dd->ic_pad[i] = icp;
            }
            const unsigned taps = icp != ic ? k / ic : 1, kk = icp != ic ? taps * icp : k;
            unsigned kpad = l.type == LAYERNORM_LAYER ? 1 : (unsigned)round_up(kk, 32);
            dd->kpad[i] = kpad;
            std::vector<float> padded((size_t)rows * kpad, 0.f);
            const float *src = (const float *)w->data;
            for (unsigned r = 0; r < rows; r++)
                for (unsigned c = 0; c < k; c++) {
                    float v = src[(size_t)r * k + c];
                    unsigned dc = icp != ic ? (c / ic) * icp + c % ic : c;
                    padded[(size_t)r * kpad + dc] = (precision == 0 && l.type != LAYERNORM_LAYER) ? round_to_tf32(v) : v;
                }
            CUDA_TRY(cudaMalloc(&dd->weight[precision][i], padded.size() * sizeof(float) + 256));
            CUDA_TRY(cudaMemcpy(dd->weight[precision][i], padded.data(), padded.size() * sizeof(float), cudaMemcpyHostToDevice));
            if (precision == 0 && l.type == CONV_LAYER && l.parent_layers[PARENT_0] && l.parent_layers[PARENT_0]->type == INPUT_LAYER && ic <= 4 &&
                l.params[WEIGHT_W] <= 8 && !dd->weight_rows[i]) {
                // second copy for the row-box staging: one 32-float chunk per filter row, (kw, channel) inside it
                const unsigned KH = l.params[WEIGHT_H], KW = l.params[WEIGHT_W];
                std::vector<float> rowsw((size_t)rows * KH * 32, 0.f);
                for (unsigned r = 0; r < rows; r++)
                    for (unsigned kh = 0; kh < KH; kh++)
                        for (unsigned kw = 0; kw < KW; kw++)
                            for (unsigned c = 0; c < ic; c++)
                                rowsw[((size_t)r * KH + kh) * 32 + kw * 4 + c] = round_to_tf32(src[(size_t)r * k + (kh * KW + kw) * ic + c]);
                CUDA_TRY(cudaMalloc(&dd->weight_rows[i], rowsw.size() * sizeof(float) + 256));
                CUDA_TRY(cudaMemcpy(dd->weight_rows[i], rowsw.data(), rowsw.size() * sizeof(float), cudaMemcpyHostToDevice));
            }
        }
        if (b && !dd->bias[i]) {
            CUDA_TRY(cudaMalloc(&dd->bias[i], (size_t)b->num_elements * sizeof(float) + 256));
            CUDA_TRY(cudaMemcpy(dd->bias[i], b->data, (size_t)b->num_elements * sizeof(float), cudaMemcpyHostToDevice));
        }
        if (a && !dd->anchors[i]) {
            CUDA_TRY(cudaMalloc(&dd->anchors[i], 8 * sizeof(float)));
            CUDA_TRY(cudaMemcpy(dd->anchors[i], a->data, 6 * sizeof(float), cudaMemcpyHostToDevice));
        }
    }
    dd->have[precision] = true;
    return 0;
}

void engine_release_dnn(aspen_dnn_t *dnn) {
    for (auto &dd : dnn->dev) {
        if (!dd) continue;
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(dd->device);
        for (int p = 0; p < 2; p++)
            for (float *ptr : dd->weight[p]) cudaFree(ptr);
        for (float *ptr : dd->bias) cudaFree(ptr);
        for (float *ptr : dd->weight_rows) cudaFree(ptr);
        for (float *ptr : dd->anchors) cudaFree(ptr);
        cudaFree(dd->emb_token);
        cudaFree(dd->emb_position);
        cudaSetDevice(prev);
        delete dd;
        dd = nullptr;
    }
}

// ---- engine --------------------------------------------------------------------------------
struct Engine {
    int device = 0;
    int precision = 0;
    int num_sms = 0;
    unsigned n_ctas = 0;
    size_t smem_bytes = 0;
    cudaStream_t stream = nullptr, side = nullptr, io = nullptr;   // compute, stop flag, host transfers
    CtrlDev *ctrl = nullptr;
    StatusHost *status_h = nullptr;   // mapped host memory
    StatusHost *status_d = nullptr;
    unsigned *queue = nullptr;
    unsigned queue_cap = 0;
    NasmDev *nasms_d = nullptr;
    unsigned nasms_cap = 0;
    std::vector<nasm_t *> in_flight;
    std::vector<nasm_t *> uploaded;   // graphs whose images (in this order) are in nasms_d
    bool running = false;
    unsigned long long stall_ns = 2000000000ull;
    unsigned long long pipe_ns = 1000000000ull;
    unsigned long long launches = 0;
    // service mode: one kernel serves pass after pass of its graphs until dse_group_stop (see scheduler.cuh)
    bool service = false;             // the group runs its graphs this way
    bool svc_live = false;            // a service kernel was launched and has not yet been seen to end
    std::vector<nasm_t *> svc_graphs; // the graphs that kernel serves
    std::vector<nasm_t *> svc_pool;   // every graph of the group's rpool that has a device image: what the next launch serves
    unsigned long long idle_ns = 20000000ull;   // the kernel leaves after this long with no pass running
    cudaEvent_t svc_armed_ev = nullptr;
    unsigned svc_ahead = 32, run_ahead = 0;   // see CtrlDev::svc_ahead: in service mode / in a launch per run
    float *xfer = nullptr;            // device staging for packed inputs / results
    unsigned long long *prof = nullptr;   // per-CTA time accounting, allocated when ASPEN_B200_PROFILE is set
    size_t xfer_bytes = 0;
};

struct DeviceNasm {
    Engine *e = nullptr;
    DeviceDnn *dd = nullptr;
    float *arena = nullptr;
    size_t arena_bytes = 0;
    std::vector<size_t> ldata_off;
    LayerDev *layers = nullptr;
    TileDev *tiles = nullptr;
    unsigned *children = nullptr, *dep = nullptr, *dep_init = nullptr, *layer_done = nullptr, *layer_tiles = nullptr, *init_ready = nullptr;
    unsigned *layers_completed = nullptr, *layer_done_init = nullptr;
    unsigned *completed_h = nullptr, *completed_d = nullptr;   // mapped flag
    void *wmaps = nullptr;
    NasmDev host;        // template; tile_base / queue_base are filled per run
    bool armed = false;  // has input, counters will be reset at the next run
    bool round_input = false;   // tensor-core path: the input is rounded to TF32 after upload
    bool ran = false;
    // service mode
    unsigned *svc_d = nullptr;                               // SVC_* words
    unsigned *svc_done_h = nullptr, *svc_done_d = nullptr;   // mapped: number of the last complete pass
    unsigned svc_armed = 0;                                  // number of the last pass the host has asked for
    unsigned n_exec = 0, n_input = 0;
    bool svc_ids = false;                                    // the last input was token ids
    bool fused_attention = false;   // some attention_v layer computes its own probabilities: the run needs the kernel that has that tile
    // Transfers next to a running graph: only DMA goes to the transfer stream (a kernel could not start while the
    // scheduler kernel holds every SM's shared memory); the scatter of a strided input and the gather of the last
    // layer's result are kernels on the compute stream, ordered around the graph's own run.
    float *in_stage = nullptr;          // packed input as uploaded, scattered into layer 0 just before the run
    int *ids_stage = nullptr;           // token ids as uploaded, gathered into layer 0 just before the run
    float *res_packed = nullptr;        // last layer gathered right after each run
    cudaEvent_t in_consumed = nullptr;  // compute stream: in_stage has been scattered
    cudaEvent_t res_ready = nullptr;    // compute stream: the run (and the gather) are complete
    bool res_valid = false;
    // A_TMA_ROWS: zero-padded [sample][PH][PW][4] copy of the input image (borders stay zero), filled after each upload
    std::vector<float *> scratch;       // transposed copies of attention value matrices (see LayerDev::vt_out)
    float *padded_in = nullptr;
    unsigned pin_ph = 0, pin_pw = 0, pin_pad = 0, pin_ic = 0, pin_ih = 0, pin_iw = 0;
};

static bool env_u64(const char *name, unsigned long long *out) {
    const char *v = getenv(name);
    if (!v || !*v) return false;
    *out = strtoull(v, nullptr, 10);
    return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

Engine *engine_create(int device, int precision, unsigned int /*num_dse_hint*/) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device >= count) {
        cudaGetLastError();
        ASPEN_ERR("no CUDA device %d (%d visible); this library has no CPU execution path\n", device, count);
        return nullptr;
    }
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        ASPEN_ERR("cannot select CUDA device %d\n", device);
        return nullptr;
    }
    if (prop.major != 10) {
        ASPEN_ERR("device %d is sm_%d%d; the kernels are built for sm_100a only\n", device, prop.major, prop.minor);
        return nullptr;
    }
    Engine *e = new Engine();
    e->device = device;
    e->precision = precision;
    e->num_sms = prop.multiProcessorCount;
    unsigned long long v;
    e->n_ctas = (unsigned)e->num_sms;
    if (env_u64("ASPEN_B200_CTAS", &v) && v > 0 && v <= (unsigned long long)e->num_sms) e->n_ctas = (unsigned)v;
    if (env_u64("ASPEN_B200_STALL_MS", &v) && v > 0) e->stall_ns = v * 1000000ull;
    if (env_u64("ASPEN_B200_PIPE_MS", &v) && v > 0) e->pipe_ns = v * 1000000ull;
    e->smem_bytes = (precision == 0 ? (size_t)tc::STAGES * tc::STAGE_BYTES + tc::EPI_BYTES + tc::RES_BYTES : 0) + sizeof(tc::Shared) + 1024;
    bool ok = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&e->side, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&e->io, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMalloc(&e->ctrl, sizeof(CtrlDev)) == cudaSuccess && cudaMemset(e->ctrl, 0, sizeof(CtrlDev)) == cudaSuccess &&
              cudaHostAlloc(&e->status_h, sizeof(StatusHost), cudaHostAllocMapped) == cudaSuccess &&
              cudaHostGetDevicePointer(&e->status_d, e->status_h, 0) == cudaSuccess;
    if (ok) {
        memset((void *)e->status_h, 0, sizeof(StatusHost));
        cudaError_t a = precision == 0
            ? cudaFuncSetAttribute(sched::scheduler_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->smem_bytes)
            : cudaFuncSetAttribute(sched::scheduler_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->smem_bytes);
        ok = a == cudaSuccess;
        if (ok && precision == 0)
            ok = cudaFuncSetAttribute(sched::scheduler_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->smem_bytes) == cudaSuccess;
        if (ok)
            ok = (precision == 0
                ? cudaFuncSetAttribute(sched::scheduler_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->smem_bytes)
                : cudaFuncSetAttribute(sched::scheduler_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->smem_bytes)) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&e->svc_armed_ev, cudaEventDisableTiming) == cudaSuccess;
        if (env_u64("ASPEN_B200_IDLE_MS", &v) && v > 0) e->idle_ns = v * 1000000ull;
        if (env_u64("ASPEN_B200_SVC_AHEAD", &v)) e->svc_ahead = (unsigned)v;
        if (env_u64("ASPEN_B200_SERVICE", &v)) e->service = v != 0;      // for programs that cannot call aspen_b200_dse_group_set_service
        if (env_u64("ASPEN_B200_RUN_AHEAD", &v)) e->run_ahead = (unsigned)v;
    }
    if (ok && getenv("ASPEN_B200_PROFILE")) {
        size_t bytes = (size_t)e->n_ctas * sched::PROF_SLOTS * sizeof(unsigned long long);
        ok = cudaMalloc(&e->prof, bytes) == cudaSuccess && cudaMemset(e->prof, 0, bytes) == cudaSuccess;
    }
    if (ok && precision == 0 && !get_encode_fn()) { ASPEN_ERR("driver has no cuTensorMapEncodeTiled\n"); ok = false; }
    if (!ok) {
        ASPEN_ERR("engine_create: CUDA setup failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        engine_destroy(e);
        return nullptr;
    }
    return e;
}

void engine_destroy(Engine *e) {
    if (!e) return;
    cudaSetDevice(e->device);
    svc_halt(e);
    if (e->stream) cudaStreamSynchronize(e->stream);
    if (e->stream) cudaStreamDestroy(e->stream);
    if (e->side) cudaStreamDestroy(e->side);
    if (e->io) cudaStreamDestroy(e->io);
    if (e->svc_armed_ev) cudaEventDestroy(e->svc_armed_ev);
    cudaFree(e->ctrl);
    if (e->status_h) cudaFreeHost((void *)e->status_h);
    cudaFree(e->queue);
    cudaFree(e->nasms_d);
    cudaFree(e->xfer);
    cudaFree(e->prof);
    delete e;
}

int engine_status(Engine *e) { return e ? (int)e->status_h->status : ASPEN_B200_ERR_CUDA; }

template <typename T>
static int to_device(T **dst, const std::vector<T> &src) {
    size_t bytes = std::max<size_t>(src.size(), 1) * sizeof(T);
    CUDA_TRY(cudaMalloc(dst, bytes));
    if (!src.empty()) CUDA_TRY(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
    return 0;
}

// Stream for host <-> device transfers of one graph.  They run on a stream of their own so that the input
// of the next graph uploads (and a finished graph's result downloads) while the scheduler kernel of
// another graph is running; only a graph that is itself still being computed makes the transfer wait for
// that run.
static cudaStream_t io_stream(Engine *e, const nasm_t *nasm) {
    if (e->service) return e->io;
    if (e->running && std::find(e->in_flight.begin(), e->in_flight.end(), nasm) != e->in_flight.end() &&
        *(volatile unsigned *)nasm->dev->completed_h == 0)
        cudaStreamSynchronize(e->stream);
    return e->io;
}

static int ensure_xfer(Engine *e, size_t bytes) {
    if (e->xfer_bytes >= bytes) return 0;
    cudaFree(e->xfer);
    e->xfer = nullptr;
    e->xfer_bytes = 0;
    CUDA_TRY(cudaMalloc(&e->xfer, bytes));
    e->xfer_bytes = bytes;
    return 0;
}

// packed [W][H] <-> strided [W][ld] activation matrix.  Small blocks; while a scheduler kernel is resident they wait
// for it (it takes all but a sliver of every SM's registers and shared memory), which stream order asks for anyway
// wherever they sit on the compute stream.
constexpr unsigned XFER_THREADS = 64;
// layer-0 matrix [pixel][ld] (already rounded) -> interior of the zero-padded [sample][PH][PW][4] copy
__global__ void fill_padded_input(float *dst, const float *src, unsigned ld, unsigned IC, unsigned IH, unsigned IW, unsigned PH, unsigned PW,
                                  unsigned pad, size_t pixels) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < pixels; i += (size_t)gridDim.x * blockDim.x) {
        const size_t b = i / ((size_t)IH * IW), r = i - b * IH * IW;
        const unsigned ih = (unsigned)(r / IW), iw = (unsigned)(r - (size_t)ih * IW);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const float *p = src + i * ld;
        v.x = p[0];
        if (IC > 1) v.y = p[1];
        if (IC > 2) v.z = p[2];
        if (IC > 3) v.w = p[3];
        reinterpret_cast<float4 *>(dst)[(b * PH + ih + pad) * PW + iw + pad] = v;
    }
}
// Token ids -> layer-0 hidden states: column t (= b * seq + s) is the id's row of the token table plus row s of the
// position table.  One 16-byte piece per thread and step; consecutive threads take consecutive pieces of a row, so
// reads of a table row and writes of a column are 128-bit and coalesced.  Ids outside the table are clamped.
__global__ void embedding_gather(float *dst, unsigned ld, const int *ids, const float *tok, const float *pos, unsigned M, unsigned seq,
                                 unsigned vocab, size_t n_tokens, int round) {
    const unsigned m4 = M >> 2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_tokens * m4; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / m4;
        const unsigned j = (unsigned)(i - t * m4) * 4u;
        int id = ids[t];
        id = id < 0 ? 0 : (id >= (int)vocab ? (int)vocab - 1 : id);
        float4 v = __ldg(reinterpret_cast<const float4 *>(tok + (size_t)id * M + j));
        if (pos) {
            const float4 p = __ldg(reinterpret_cast<const float4 *>(pos + (size_t)(t % seq) * M + j));
            v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        if (round) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
        *reinterpret_cast<float4 *>(dst + t * ld + j) = v;
    }
}
__global__ void unpack_columns(float *dst, const float *src, unsigned H, unsigned ld, size_t n, int round) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        size_t w = i / H;
        unsigned h = (unsigned)(i - w * H);
        dst[w * ld + h] = round ? tf32_round(src[i]) : src[i];
    }
}
__global__ void round_tf32_inplace(float *p, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = tf32_round(p[i]);
}
__global__ void pack_columns(float *dst, const float *src, unsigned H, unsigned ld, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        size_t w = i / H;
        unsigned h = (unsigned)(i - w * H);
        dst[i] = src[w * ld + h];
    }
}

static void fill_layer(const nasm_t *nasm, const DeviceNasm *dn, unsigned i, int precision, LayerDev &L, int wmap_idx) {
    const nasm_ldata_t &ld = nasm->ldata[i];
    const aspen_layer_t &l = *ld.layer;
    const unsigned *p = l.params;
    memset(&L, 0, sizeof L);
    L.type = l.type;
    L.act = l.activation;
    L.out = (float *)((char *)dn->arena + dn->ldata_off[i]);
    L.ldc = ld.out_mat_stride; L.H = ld.out_mat_dims[OUT_H]; L.W = ld.out_mat_dims[OUT_W];
    unsigned p0 = ld.parent_ldata_idx_arr[PARENT_0], p1 = ld.parent_ldata_idx_arr[PARENT_1];
    if (p0 != (unsigned)-1) {
        L.in0 = (const float *)((char *)dn->arena + dn->ldata_off[p0]);
        L.ld0 = nasm->ldata[p0].out_mat_stride; L.H0 = nasm->ldata[p0].out_mat_dims[OUT_H];
    }
    if (p1 != (unsigned)-1) {
        L.in1 = (const float *)((char *)dn->arena + dn->ldata_off[p1]);
        L.ld1 = nasm->ldata[p1].out_mat_stride; L.H1 = nasm->ldata[p1].out_mat_dims[OUT_H];
    }
    L.weight = dn->dd->weight[precision][i];
    L.bias = dn->dd->bias[i];
    L.anchors = dn->dd->anchors[i];
    L.rows = layer_weight_rows(&l);
    L.K = layer_contraction_k(&l);
    L.Kpad = dn->dd->kpad[i];
    L.IC = p[IN_C]; L.IH = p[IN_H]; L.IW = p[IN_W]; L.OH = p[OUT_H]; L.OW = p[OUT_W];
    L.KH = p[WEIGHT_H]; L.KW = p[WEIGHT_W]; L.stride = p[STRIDE] ? p[STRIDE] : 1; L.pad = p[PADDING];
    if (l.type == FC_LAYER) { L.KH = p[IN_H]; L.KW = p[IN_W]; L.OH = 1; L.OW = 1; L.stride = 1; L.pad = 0; }
    if (dn->dd->ic_pad[i] && L.ld0 >= dn->dd->ic_pad[i]) { L.IC = dn->dd->ic_pad[i]; L.K = L.KH * L.KW * L.IC; }
    L.seq = nasm->tr_seq_len; L.heads = p[NUM_HEAD]; L.hd = p[NUM_HEAD] ? p[NUM_HIDDEN] / p[NUM_HEAD] : 0; L.masked = p[MASKED];
    L.p_out_c = p[OUT_C]; L.p_in_c = p[IN_C]; L.p_stride = p[STRIDE];
    L.wmap = wmap_idx;
    L.resmap = -1;
    L.bw = 128;
    switch (l.type) {
        case CONV_LAYER: case FC_LAYER: L.a_vec4 = (L.IC % 4 == 0) && (L.ld0 % 4 == 0); break;
        case MATMUL_LAYER: L.a_vec4 = (L.K % 4 == 0) && (L.ld0 % 4 == 0); break;
        case K_ATTENTION_LAYER: L.a_vec4 = (L.hd % 4 == 0) && (L.ld0 % 4 == 0) && (L.ld1 % 4 == 0); break;
        case V_ATTENTION_LAYER: L.a_vec4 = (L.seq % 4 == 0) && (L.ld0 % 4 == 0); break;
        default: L.a_vec4 = 0; break;
    }
}

static void free_device_nasm(DeviceNasm *dn) {
    if (!dn) return;
    cudaFree(dn->arena); cudaFree(dn->layers); cudaFree(dn->tiles); cudaFree(dn->children); cudaFree(dn->dep);
    cudaFree(dn->dep_init); cudaFree(dn->layer_done); cudaFree(dn->layer_tiles); cudaFree(dn->init_ready);
    cudaFree(dn->layers_completed); cudaFree(dn->layer_done_init); cudaFree(dn->wmaps);
    if (dn->completed_h) cudaFreeHost(dn->completed_h);
    if (dn->svc_done_h) cudaFreeHost(dn->svc_done_h);
    cudaFree(dn->svc_d);
    cudaFree(dn->in_stage); cudaFree(dn->ids_stage); cudaFree(dn->res_packed); cudaFree(dn->padded_in);
    for (float *p : dn->scratch) cudaFree(p);
    if (dn->in_consumed) cudaEventDestroy(dn->in_consumed);
    if (dn->res_ready) cudaEventDestroy(dn->res_ready);
    delete dn;
}

static int build_device_nasm(Engine *e, nasm_t *nasm) {
    DeviceNasm *dn = new DeviceNasm();
    dn->e = e;
    nasm->dev = dn;
    if (upload_weights(nasm->dnn, e->device, e->precision, &dn->dd) != 0) return -1;
    // activation arena: one region per layer (no reuse: every layer output stays readable)
    dn->ldata_off.resize(nasm->num_ldata);
    size_t off = 0;
    for (unsigned i = 0; i < nasm->num_ldata; i++) {
        dn->ldata_off[i] = off;
        off += round_up(nasm->ldata[i].out_mat_mem_size + 64, 256);
    }
    dn->arena_bytes = off + 4096;
    CUDA_TRY(cudaMalloc(&dn->arena, dn->arena_bytes));
    CUDA_TRY(cudaMemsetAsync(dn->arena, 0, dn->arena_bytes, e->stream));

    // layers + tensor maps (weights and, where the access pattern allows it, the parents' activations)
    std::vector<LayerDev> layers(nasm->num_ldata);
    std::vector<CUtensorMap> maps;
    auto add_map = [&](const void *base, cuuint64_t inner, cuuint64_t outer, cuuint64_t stride_bytes, cuuint32_t box_rows) -> int {
        CUtensorMap m;
        cuuint64_t dims[2] = {inner, outer};
        cuuint64_t strides[1] = {stride_bytes};
        cuuint32_t box[2] = {32, box_rows}, estr[2] = {1, 1};
        CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { ASPEN_ERR("cuTensorMapEncodeTiled failed (%d)\n", (int)r); return -2; }
        maps.push_back(m);
        return (int)maps.size() - 1;
    };
    // 3-D map of the padded input copy: (32 floats of a row, output pixel = `stride` input pixels apart, row)
    // Eight consecutive maps, the j-th with a box of 16 j pixels.  Returns the index of the first, or -2 when the driver
    // does not take such (overlapping) maps: the layer then keeps the gather.
    auto add_rows_map = [&](const void *base, unsigned OW, unsigned stride, unsigned PW, cuuint64_t rows_total) -> int {
        const size_t first = maps.size();
        for (unsigned j = 1; j <= 8; j++) {
            CUtensorMap m;
            cuuint64_t dims[3] = {32, OW, rows_total};
            cuuint64_t strides[2] = {(cuuint64_t)stride * 16, (cuuint64_t)PW * 16};
            cuuint32_t box[3] = {32, std::min(16 * j, OW), 1}, estr[3] = {1, 1, 1};
            CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims, strides, box, estr,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) { maps.resize(first); return -2; }
            maps.push_back(m);
        }
        return (int)first;
    };
    // Maps of the im2col staging (A_TMA_IM2COL): the parent as (channel, iw, ih, sample), element stride = convolution
    // stride on iw and ih.  Index L - 1: a run of L pixels of one output row; index OW + k - 2: k whole output rows.
    auto add_im2col_maps = [&](const void *base, unsigned C, unsigned IW, unsigned IH, unsigned B, unsigned ld, unsigned stride, unsigned OW,
                               unsigned OH) -> int {
        const size_t first = maps.size();
        const unsigned kmax = std::max(1u, std::min(OH, 128u / OW));
        for (unsigned idx = 0; idx < OW + kmax - 1; idx++) {
            const unsigned len = idx < OW ? idx + 1 : OW, rows = idx < OW ? 1 : idx - OW + 2;
            CUtensorMap m;
            cuuint64_t dims[4] = {C, IW, IH, B};
            cuuint64_t strides[3] = {(cuuint64_t)ld * 4, (cuuint64_t)IW * ld * 4, (cuuint64_t)IH * IW * ld * 4};
            cuuint32_t box[4] = {32, len * stride, rows * stride, 1}, estr[4] = {1, stride, stride, 1};
            CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(base), dims, strides, box, estr,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) { maps.resize(first); return -2; }
            maps.push_back(m);
        }
        if (OW * OH <= 128) {   // last map: whole samples (a block of conv_block_width pixels)
            CUtensorMap m;
            cuuint64_t dims[4] = {C, IW, IH, B};
            cuuint64_t strides[3] = {(cuuint64_t)ld * 4, (cuuint64_t)IW * ld * 4, (cuuint64_t)IH * IW * ld * 4};
            cuuint32_t box[4] = {32, OW * stride, OH * stride, 128 / (OW * OH)}, estr[4] = {1, stride, stride, 1};
            CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(base), dims, strides, box, estr,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) { maps.resize(first); return -2; }
            maps.push_back(m);
        }
        return (int)first;
    };
    unsigned long long im2col_mode = 1;   // 0: off, 1: convolutions that would otherwise gather, 2: also the stride-1 "same" ones
    env_u64("ASPEN_B200_IM2COL", &im2col_mode);
    const char *no_rows = getenv("ASPEN_B200_NO_ROW_BOXES");
    for (unsigned i = 0; i < nasm->num_ldata; i++) {
        const aspen_layer_t &l = *nasm->ldata[i].layer;
        LayerDev &L = layers[i];
        fill_layer(nasm, dn, i, e->precision, L, -1);
        L.amap = -1;
        L.a_kind = tc::A_GATHER;
        L.b_kind = tc::B_GATHER;
        if (e->precision != 0) continue;
        const bool gemm_w = l.type == CONV_LAYER || l.type == FC_LAYER || l.type == MATMUL_LAYER;
        const unsigned p0 = nasm->ldata[i].parent_ldata_idx_arr[PARENT_0], p1 = nasm->ldata[i].parent_ldata_idx_arr[PARENT_1];
        const cuuint64_t W0 = p0 != (unsigned)-1 ? nasm->ldata[p0].out_mat_dims[OUT_W] : 0;
        // Row-box staging of an input convolution (see tiles_tc.cuh, A_TMA_ROWS): decided first, it changes the
        // weight layout the weight map is made from.
        bool rows_kind = false;
        if (l.type == CONV_LAYER && p0 == 0 && dn->dd->weight_rows[i] && !dn->padded_in && !(no_rows && atoi(no_rows) != 0) &&
            L.OW % 16 == 0 && nasm->ldata[i].out_mat_dims[OUT_W] % 128 == 0 && nasm->ldata[i].ninst_tile_dims[OUT_W] % 128 == 0) {
            const unsigned s_ = L.stride, pad = L.pad;
            const unsigned PW = std::max(L.IW + 2 * pad, s_ * (L.OW - 1) + 8), PH = std::max(L.IH + 2 * pad, s_ * (L.OH - 1) + L.KH);
            const size_t bytes = (size_t)nasm->batch_size * PH * PW * 4 * sizeof(float);
            CUDA_TRY(cudaMalloc(&dn->padded_in, bytes + 256));
            CUDA_TRY(cudaMemsetAsync(dn->padded_in, 0, bytes + 256, e->stream));
            const int m = add_rows_map(dn->padded_in, L.OW, s_, PW, (cuuint64_t)nasm->batch_size * PH);
            if (m >= 0) {
                dn->pin_ph = PH; dn->pin_pw = PW; dn->pin_pad = pad; dn->pin_ic = l.params[IN_C]; dn->pin_ih = L.IH; dn->pin_iw = L.IW;
                rows_kind = true;
                L.a_kind = tc::A_TMA_ROWS;
                L.amap = m;
                L.PH = PH;
                L.weight = dn->dd->weight_rows[i];
                L.Kpad = L.KH * 32;
                L.K = L.Kpad;
            } else {
                cudaFree(dn->padded_in);
                dn->padded_in = nullptr;
            }
        }
        if (gemm_w) {
            L.b_kind = tc::B_TMA;
            L.wmap = add_map(L.weight, L.Kpad, layer_weight_rows(&l), (cuuint64_t)L.Kpad * sizeof(float), 64);
            if (L.wmap < 0) return -1;
        }
        const bool aligned0 = L.ld0 % 4 == 0;
        if (rows_kind) {
            // operands set above
        } else if (l.type == MATMUL_LAYER && aligned0 && L.K % 4 == 0) {
            L.a_kind = tc::A_TMA;
            L.amap = add_map(L.in0, L.H0, W0, (cuuint64_t)L.ld0 * sizeof(float), 128);
        } else if (l.type == CONV_LAYER && aligned0 && L.IC % 4 == 0 && L.KH == 1 && L.KW == 1 && L.stride == 1 && L.pad == 0) {
            L.a_kind = tc::A_TMA;
            L.amap = add_map(L.in0, L.H0, W0, (cuuint64_t)L.ld0 * sizeof(float), 128);
        } else if (l.type == CONV_LAYER && aligned0 && L.IC % 32 == 0 && L.stride == 1 && L.OH == L.IH && L.OW == L.IW && L.KH == L.KW &&
                   2 * L.pad + 1 == L.KH && im2col_mode != 2) {
            L.a_kind = tc::A_TMA_FIXUP;
            L.amap = add_map(L.in0, L.H0, W0, (cuuint64_t)L.ld0 * sizeof(float), 128);
        } else if (l.type == CONV_LAYER && aligned0 && L.IC % 32 == 0 && L.IC == L.H0 && im2col_mode != 0 && L.OW * L.stride <= 256 &&
                   L.stride <= 8 && L.OW <= 128 && L.KH * L.KW * L.IC == L.K) {
            const int m = add_im2col_maps(L.in0, L.IC, L.IW, L.IH, nasm->batch_size, L.ld0, L.stride, L.OW, L.OH);
            if (m >= 0) {
                L.a_kind = tc::A_TMA_IM2COL;
                L.amap = m;
                // Tiles made of blocks of whole output rows / samples (the tiler does that for these layers when the column
                // quantum is 128): each block is then one box.
                const unsigned bw = conv_block_width(L.OW, L.OH), kmax = std::max(1u, std::min(L.OH, 128u / L.OW));
                if (bw != 128 && conv_uses_row_blocks(&l) && nasm->ldata[i].ninst_tile_dims[OUT_W] % bw == 0) {
                    L.bw = bw;
                    L.one_box = L.OW * L.OH <= 128 ? L.OW + kmax - 1 : L.OW + bw / L.OW - 2;
                }
            }
        } else if (l.type == FC_LAYER && L.ld0 == L.IC && L.K % 4 == 0) {
            L.a_kind = tc::A_TMA;   // a sample's NHWC activations are one contiguous row of K values
            L.amap = add_map(L.in0, L.K, nasm->batch_size, (cuuint64_t)L.IH * L.IW * L.ld0 * sizeof(float), 128);
        } else if (l.type == K_ATTENTION_LAYER) {
            if (!L.a_vec4 || L.seq > tc::TMEM_COLS) {
                ASPEN_ERR("attention_k layer %u: head size must be a multiple of 4 and seq <= %u on the tensor-core path\n", i, tc::TMEM_COLS);
                return -1;
            }
            if (L.hd % 32 == 0) {
                L.a_kind = tc::A_TMA;
                L.amap = add_map(L.in0, L.H0, W0, (cuuint64_t)L.ld0 * sizeof(float), 128);
                L.b_kind = tc::B_TMA_ACT;
                L.wmap = add_map(L.in1, L.H1, nasm->ldata[p1].out_mat_dims[OUT_W], (cuuint64_t)L.ld1 * sizeof(float), 64);
                if (L.wmap < 0) return -1;
            }
        } else if (l.type == V_ATTENTION_LAYER) {
            L.b_kind = tc::B_TRANSPOSED;
            if (aligned0) {
                L.a_kind = tc::A_TMA;
                L.amap = add_map(L.in0, L.H0, W0, (cuuint64_t)L.ld0 * sizeof(float), 128);
            }
            // The value operand W(m, k) = V[token k][feature m] is the transpose of how the value projection stores its
            // output.  Where that projection is a tensor-core layer of this graph (it precedes this one), it writes a
            // second, transposed copy into scratch memory, which TMA then stages like any K-major operand; otherwise the
            // worker threads gather it element by element.
            const char *no_vt = getenv("ASPEN_B200_NO_VT");
            const LAYER_TYPE pt = p1 != (unsigned)-1 ? nasm->ldata[p1].layer->type : NO_LAYER_TYPE;
            if (p1 != (unsigned)-1 && p1 < i && p1 != 0 && (pt == MATMUL_LAYER || pt == CONV_LAYER) && L.seq % 4 == 0 && !layers[p1].vt_out &&
                !(no_vt && atoi(no_vt) != 0)) {
                const size_t W1 = nasm->ldata[p1].out_mat_dims[OUT_W], ldt = round_up(W1, 32);
                float *vt = nullptr;
                CUDA_TRY(cudaMalloc(&vt, (size_t)L.H1 * ldt * sizeof(float) + 256));
                dn->scratch.push_back(vt);
                CUDA_TRY(cudaMemsetAsync(vt, 0, (size_t)L.H1 * ldt * sizeof(float) + 256, e->stream));
                const int m = add_map(vt, W1, L.H1, (cuuint64_t)ldt * sizeof(float), 64);
                if (m >= 0) {
                    layers[p1].vt_out = vt;
                    layers[p1].vt_ld = (unsigned)ldt;
                    L.b_kind = tc::B_TMA_ACT;
                    L.wmap = m;
                }
            }
        }
        if (L.a_kind != tc::A_GATHER && L.amap < 0) return -1;
    }
    if (e->precision == 0) {
        for (unsigned i = 0; i < nasm->num_ldata; i++) {
            const LAYER_TYPE t = nasm->ldata[i].layer->type;
            if (t == CONV_LAYER || t == FC_LAYER || t == MATMUL_LAYER || t == K_ATTENTION_LAYER || t == V_ATTENTION_LAYER)
                for (int k = PARENT_0; k <= PARENT_1; k++) {
                    unsigned par = nasm->ldata[i].parent_ldata_idx_arr[k];
                    if (par != (unsigned)-1) layers[par].round_out = 1;
                }
        }
    }
    dn->round_input = layers[0].round_out != 0;
    // Attention fusion (tensor-core path): an attention_v layer whose probabilities come from an attention_k layer that
    // nothing else reads computes them itself, per (sample, head, block of queries), and the seq x seq matrix never goes
    // to memory (ref src/tiled_kernels.c:784-1038 are two layers).  Needs head sizes of 32 or 64, the TMA staging of
    // queries, keys and the transposed values, and one head per tile row.  Where every hidden state has to stay readable
    // the tile also writes the probabilities, which it can only do when all keys fit one group of 128.
    // OFF unless ASPEN_B200_ATTN_FUSE=1: the fused tile itself takes 13 us where the two tiles it replaces take 20
    // (BERT-base, 128 x 128 x 64 per head), but the kernel instantiation that contains it runs every other tile type about
    // 1.5 x slower (its register allocation spills on the common path, and with 176 KB of shared memory per CTA little L1
    // is left to absorb spills), a net loss for now.  Not for a group in service mode (that kernel has no fused tile).
    std::vector<unsigned char> attn_bypassed(nasm->num_ldata, 0);
    const char *want_attn = getenv("ASPEN_B200_ATTN_FUSE");
    if (e->precision == 0 && !e->service && want_attn && atoi(want_attn) != 0) {
        for (unsigned i = 1; i < nasm->num_ldata; i++) {
            if (nasm->ldata[i].layer->type != V_ATTENTION_LAYER) continue;
            LayerDev &V = layers[i];
            const unsigned k = nasm->ldata[i].parent_ldata_idx_arr[PARENT_0];
            if (k == (unsigned)-1 || nasm->ldata[k].layer->type != K_ATTENTION_LAYER) continue;
            const LayerDev &K = layers[k];
            bool only_reader = true;
            for (unsigned j = 1; j < nasm->num_ldata; j++)
                if (j != i && (nasm->ldata[j].parent_ldata_idx_arr[PARENT_0] == k || nasm->ldata[j].parent_ldata_idx_arr[PARENT_1] == k)) only_reader = false;
            const bool keep = keep_hidden_states();
            if (!only_reader || k == nasm->num_ldata - 1) continue;
            if (V.b_kind != tc::B_TMA_ACT || V.a_kind != tc::A_TMA || K.a_kind != tc::A_TMA || K.b_kind != tc::B_TMA_ACT) continue;
            if ((V.hd != 32 && V.hd != 64) || K.hd != V.hd || K.heads != V.heads) continue;
            if (nasm->ldata[i].ninst_tile_dims[OUT_H] != V.hd || nasm->ldata[i].ninst_tile_dims[OUT_W] > 128 || V.seq % nasm->ldata[i].ninst_tile_dims[OUT_W] != 0) continue;
            if (keep && V.seq > 128) continue;
            V.att_fused = 1;
            V.att_qmap = K.amap;
            V.att_kmap = K.wmap;
            V.masked = K.masked;
            if (keep) { V.att_p_out = K.out; V.att_p_ld = K.ldc; V.att_p_round = K.round_out; }
            attn_bypassed[k] = 1;
            dn->fused_attention = true;
        }
    }
    // Residual fusion (tensor-core path): a residual layer whose later parent is a convolution or a matmul
    // is computed in that parent's epilogue, which then needs the earlier parent's tiles of the same region
    // (fused_other[producer] = that layer).  The residual layer's own tiles stay in the graph and only pass
    // completion on.  ASPEN_B200_NO_FUSE=1 keeps the layers separate.
    std::vector<unsigned> fused_other(nasm->num_ldata, (unsigned)-1);
    std::vector<unsigned char> written_by_parents(nasm->num_ldata, 0);
    const char *no_fuse = getenv("ASPEN_B200_NO_FUSE");
    if (e->precision == 0 && !(no_fuse && atoi(no_fuse) != 0)) {
        for (unsigned i = 1; i < nasm->num_ldata; i++) {
            if (nasm->ldata[i].layer->type != RESIDUAL_LAYER) continue;
            const unsigned a = nasm->ldata[i].parent_ldata_idx_arr[PARENT_0], b = nasm->ldata[i].parent_ldata_idx_arr[PARENT_1];
            if (a == (unsigned)-1 || b == (unsigned)-1 || a == b) continue;
            const unsigned hi = std::max(a, b), lo = std::min(a, b);
            const LAYER_TYPE t = nasm->ldata[hi].layer->type;
            if (lo == 0 || (t != CONV_LAYER && t != MATMUL_LAYER) || layers[hi].res_out) continue;
            const nasm_ldata_t &R = nasm->ldata[i], &P = nasm->ldata[hi], &Q = nasm->ldata[lo];
            if (P.out_mat_dims[OUT_H] != R.out_mat_dims[OUT_H] || P.out_mat_dims[OUT_W] != R.out_mat_dims[OUT_W] ||
                Q.out_mat_dims[OUT_H] != R.out_mat_dims[OUT_H] || Q.out_mat_dims[OUT_W] != R.out_mat_dims[OUT_W])
                continue;
            LayerDev &L = layers[hi];
            L.res_in = layers[lo].out; L.res_ld_in = layers[lo].ldc;
            L.res_out = layers[i].out; L.res_ld_out = layers[i].ldc;
            L.res_act = layers[i].act; L.res_round = layers[i].round_out;
            // the other operand reaches the epilogue as 32 x 32 boxes by TMA (falls back to plain loads if the driver refuses the map)
            const char *no_res_tma = getenv("ASPEN_B200_NO_RES_TMA");
            if (layers[lo].ldc % 4 == 0 && !(no_res_tma && atoi(no_res_tma) != 0)) {
                const int m = add_map(layers[lo].out, Q.out_mat_dims[OUT_H], Q.out_mat_dims[OUT_W], (cuuint64_t)layers[lo].ldc * sizeof(float), 32);
                L.resmap = m >= 0 ? m : -1;
            }
            // The producer's own (pre-add) output: the reference frees it as soon as the residual layer has read it
            // (src/dse.c:84-92).  When nothing else reads it and the caller has not asked for every hidden state,
            // it is not written at all.
            bool only_reader = true;
            for (unsigned j = 1; j < nasm->num_ldata; j++)
                if (j != i && (nasm->ldata[j].parent_ldata_idx_arr[PARENT_0] == hi || nasm->ldata[j].parent_ldata_idx_arr[PARENT_1] == hi)) only_reader = false;
            L.res_elide = (!keep_hidden_states() && only_reader && hi != nasm->num_ldata - 1) ? 1u : 0u;
            fused_other[hi] = lo;
            written_by_parents[i] = 1;
        }
    }
    if (to_device(&dn->layers, layers) != 0) return -1;
    {
        size_t bytes = std::max<size_t>(maps.size(), 1) * sizeof(CUtensorMap);
        CUDA_TRY(cudaMalloc(&dn->wmaps, bytes));
        if (!maps.empty()) CUDA_TRY(cudaMemcpy(dn->wmaps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice));
    }

    // tiles, children (CSR), counters.  A tile's count to reach is the length of its parent list plus
    // the true-dependency supplement; the edges walked at completion are the host child lists (as the
    // reference walks child_ninst_arr, src/dse.c:372-375) plus the supplement.  For a generated graph the
    // two agree; a file whose lists disagree yields a tile that never becomes ready, which the
    // scheduler reports as a stall.
    const unsigned n = nasm->num_ninst;
    std::vector<TileDev> tiles(n);
    std::vector<std::vector<unsigned>> kids(n);
    std::vector<unsigned> dep_init(n, 0), init_ready, layer_tiles(nasm->num_ldata);
    const unsigned n_input = nasm->ldata[0].num_ninst;
    for (unsigned t = 0; t < n; t++) {
        const ninst_t &ni = nasm->ninst[t];
        TileDev &T = tiles[t];
        T.layer = (unsigned)(ni.ldata - nasm->ldata.data());
        T.pos_h = ni.out_mat_pos[OUT_H]; T.pos_w = ni.out_mat_pos[OUT_W];
        T.tile_h = ni.tile_dims[OUT_H]; T.tile_w = ni.tile_dims[OUT_W];
        T.need = (unsigned)(ni.parent_ninst_idx.size() + ni.extra_parent_idx.size());
        T.flags = (written_by_parents[T.layer] || attn_bypassed[T.layer]) ? TILE_WRITTEN_BY_PARENTS : 0u;
        if (fused_other[T.layer] != (unsigned)-1) {
            // the fused residual reads the other parent over this tile's own region: tiles of that layer's grid
            // (rows fastest) that overlap it become parents too
            const nasm_ldata_t &Q = nasm->ldata[fused_other[T.layer]];
            const unsigned qh = Q.ninst_tile_dims[OUT_H], qw = Q.ninst_tile_dims[OUT_W];
            const unsigned per_col = (Q.out_mat_dims[OUT_H] + qh - 1) / qh;
            for (unsigned cw = T.pos_w / qw; cw <= (T.pos_w + T.tile_w - 1) / qw; cw++)
                for (unsigned ch = T.pos_h / qh; ch <= (T.pos_h + T.tile_h - 1) / qh; ch++) {
                    const unsigned par = Q.ninst_start + cw * per_col + ch;
                    if (par >= Q.ninst_start + Q.num_ninst || par >= t) { ASPEN_ERR("fused residual: tile %u has no valid producer tile\n", t); return -1; }
                    kids[par].push_back(t);
                    T.need++;
                    if (par < n_input) dep_init[t]++;
                }
        }
        for (int pass = 0; pass < 2; pass++)
            for (unsigned par : (pass == 0 ? ni.parent_ninst_idx : ni.extra_parent_idx)) {
                if (par >= n || par >= t) { ASPEN_ERR("tile %u lists parent %u that does not precede it\n", t, par); return -1; }
                if (pass == 1) kids[par].push_back(t);
                if (par < n_input) dep_init[t]++;
            }
        for (unsigned child : ni.child_ninst_idx) {
            if (child >= n || child <= t) { ASPEN_ERR("tile %u lists child %u that does not follow it\n", t, child); return -1; }
            kids[t].push_back(child);
        }
        if (t >= n_input && T.need == 0) { ASPEN_ERR("tile %u of layer %u has no parents and can never run\n", t, T.layer); return -1; }
    }
    // Tiles whose values their parents write (fused residual layers) are taken out of the device graph: each of their
    // parent edges is replaced by edges to their children, and they count as complete from the start.  Without this
    // every such tile costs a pass through the ready queue and a completion on some CTA.  ASPEN_B200_KEEP_NOOP_TILES=1
    // leaves them in (the scheduler then completes them when they become ready).
    std::vector<unsigned> layer_done_init(nasm->num_ldata, 0);
    layer_done_init[0] = n_input;
    unsigned n_bypassed = 0;
    const char *keep_noop = getenv("ASPEN_B200_KEEP_NOOP_TILES");
    if (!(keep_noop && atoi(keep_noop) != 0)) {
        std::vector<std::vector<unsigned>> pars(n);
        for (unsigned p = 0; p < n; p++)
            for (unsigned c : kids[p]) pars[c].push_back(p);
        for (unsigned t = n_input; t < n; t++) {
            if (!(tiles[t].flags & TILE_WRITTEN_BY_PARENTS) || pars[t].empty() || pars[t].size() != tiles[t].need) continue;
            bool input_parent = false;
            for (unsigned p : pars[t]) input_parent |= p < n_input;
            if (input_parent) continue;
            for (unsigned c : kids[t]) {                       // one edge t -> c becomes the edges p -> c
                tiles[c].need += (unsigned)pars[t].size() - 1u;
                auto it = std::find(pars[c].begin(), pars[c].end(), t);
                if (it != pars[c].end()) pars[c].erase(it);
                for (unsigned p : pars[t]) { kids[p].push_back(c); pars[c].push_back(p); }
            }
            for (unsigned p : pars[t]) kids[p].erase(std::remove(kids[p].begin(), kids[p].end(), t), kids[p].end());
            kids[t].clear();
            pars[t].clear();
            tiles[t].need = 0xffffffffu;                       // never reached
            layer_done_init[tiles[t].layer]++;
            n_bypassed++;
        }
    }
    unsigned layers_done_init = 0;
    for (unsigned i = 0; i < nasm->num_ldata; i++) layers_done_init += layer_done_init[i] == nasm->ldata[i].num_ninst ? 1u : 0u;
    for (unsigned t = n_input; t < n; t++)
        if (tiles[t].need != 0xffffffffu && dep_init[t] == tiles[t].need) init_ready.push_back(t);
    std::vector<unsigned> children;   // pairs: (child tile, count that child waits for)
    for (unsigned t = 0; t < n; t++) {
        tiles[t].child_off = (unsigned)(children.size() / 2);
        tiles[t].child_cnt = (unsigned)kids[t].size();
        for (unsigned c : kids[t]) { children.push_back(c); children.push_back(tiles[c].need); }
    }
    for (unsigned i = 0; i < nasm->num_ldata; i++) layer_tiles[i] = nasm->ldata[i].num_ninst;
    std::vector<unsigned> zeros(std::max(n, nasm->num_ldata), 0);
    if (to_device(&dn->tiles, tiles) != 0 || to_device(&dn->children, children) != 0 || to_device(&dn->dep_init, dep_init) != 0 ||
        to_device(&dn->init_ready, init_ready) != 0 || to_device(&dn->layer_tiles, layer_tiles) != 0 ||
        to_device(&dn->layer_done_init, layer_done_init) != 0)
        return -1;
    CUDA_TRY(cudaMalloc(&dn->dep, std::max<size_t>(n, 1) * sizeof(unsigned)));
    CUDA_TRY(cudaMalloc(&dn->layer_done, nasm->num_ldata * sizeof(unsigned)));
    CUDA_TRY(cudaMalloc(&dn->layers_completed, sizeof(unsigned)));
    CUDA_TRY(cudaHostAlloc(&dn->completed_h, sizeof(unsigned), cudaHostAllocMapped));
    *dn->completed_h = 0;
    CUDA_TRY(cudaHostGetDevicePointer(&dn->completed_d, dn->completed_h, 0));
    CUDA_TRY(cudaHostAlloc(&dn->svc_done_h, sizeof(unsigned), cudaHostAllocMapped));
    *dn->svc_done_h = 0;
    CUDA_TRY(cudaHostGetDevicePointer(&dn->svc_done_d, dn->svc_done_h, 0));
    CUDA_TRY(cudaMalloc(&dn->svc_d, 4 * sizeof(unsigned)));
    CUDA_TRY(cudaMemset(dn->svc_d, 0, 4 * sizeof(unsigned)));
    dn->n_exec = n - n_bypassed;
    dn->n_input = n_input;

    {
        const nasm_ldata_t &l0 = nasm->ldata[0], &ll = nasm->ldata[nasm->num_ldata - 1];
        if (l0.out_mat_stride != l0.out_mat_dims[OUT_H])
            CUDA_TRY(cudaMalloc(&dn->in_stage, std::max<size_t>((size_t)l0.out_mat_dims[OUT_H] * l0.out_mat_dims[OUT_W], 1) * sizeof(float)));
        if (ll.out_mat_stride != ll.out_mat_dims[OUT_H])
            CUDA_TRY(cudaMalloc(&dn->res_packed, std::max<size_t>((size_t)ll.out_mat_dims[OUT_H] * ll.out_mat_dims[OUT_W], 1) * sizeof(float)));
        CUDA_TRY(cudaEventCreateWithFlags(&dn->in_consumed, cudaEventDisableTiming));
        CUDA_TRY(cudaEventCreateWithFlags(&dn->res_ready, cudaEventDisableTiming));
    }
    NasmDev &H = dn->host;
    memset(&H, 0, sizeof H);
    H.layers = dn->layers; H.tiles = dn->tiles; H.children = dn->children; H.dep = dn->dep; H.dep_init = dn->dep_init;
    H.layer_done = dn->layer_done; H.layer_tiles = dn->layer_tiles; H.init_ready = dn->init_ready;
    H.layers_completed = dn->layers_completed; H.completed = dn->completed_d; H.wmaps = dn->wmaps;
    H.n_tiles = n; H.n_layers = nasm->num_ldata; H.n_init = (unsigned)init_ready.size(); H.n_input_tiles = n_input + n_bypassed;
    H.layer_done_init = dn->layer_done_init; H.layers_done_init = layers_done_init;
    return 0;
}

int engine_set_input(nasm_t *nasm, const void *input_host) {
    DeviceNasm *dn = nasm->dev;
    if (!dn) return -1;
    Engine *e = dn->e;
    CUDA_TRY(cudaSetDevice(e->device));
    const nasm_ldata_t &l0 = nasm->ldata[0];
    const size_t n = (size_t)l0.out_mat_dims[OUT_H] * l0.out_mat_dims[OUT_W];
    float *dst = (float *)((char *)dn->arena + dn->ldata_off[0]);
    cudaStream_t io = io_stream(e, nasm);
    dn->res_valid = false;
    if (!input_host) {
        // no input: layer 0 is cleared, on the compute stream, ahead of the graph's next run
        CUDA_TRY(cudaMemsetAsync(dst, 0, l0.out_mat_mem_size, e->stream));
        if (dn->padded_in) CUDA_TRY(cudaMemsetAsync(dn->padded_in, 0, (size_t)nasm->batch_size * dn->pin_ph * dn->pin_pw * 4 * sizeof(float), e->stream));
        return 0;
    }
    const unsigned blocks = (unsigned)std::min<size_t>((n + XFER_THREADS - 1) / XFER_THREADS, 16384);
    if (dn->in_stage) {
        // DMA into the staging copy (after the previous scatter has read it), then the scatter on the compute stream
        CUDA_TRY(cudaStreamWaitEvent(io, dn->in_consumed, 0));
        CUDA_TRY(cudaMemcpyAsync(dn->in_stage, input_host, n * sizeof(float), cudaMemcpyHostToDevice, io));
        // The caller may reuse its buffer as soon as we return (the reference copies synchronously).
        CUDA_TRY(cudaStreamSynchronize(io));
        unpack_columns<<<blocks, XFER_THREADS, 0, e->stream>>>(dst, dn->in_stage, l0.out_mat_dims[OUT_H], l0.out_mat_stride, n, dn->round_input ? 1 : 0);
        e->launches++;
        CUDA_TRY(cudaGetLastError());
        CUDA_TRY(cudaEventRecord(dn->in_consumed, e->stream));
    } else {
        CUDA_TRY(cudaMemcpyAsync(dst, input_host, n * sizeof(float), cudaMemcpyHostToDevice, io));
        CUDA_TRY(cudaStreamSynchronize(io));
        if (dn->round_input) {   // packed layout: round in place (the strided path rounds while scattering)
            round_tf32_inplace<<<blocks, XFER_THREADS, 0, e->stream>>>(dst, n);
            e->launches++;
            CUDA_TRY(cudaGetLastError());
        }
    }
    if (dn->padded_in) {
        const size_t pixels = l0.out_mat_dims[OUT_W];
        fill_padded_input<<<(unsigned)std::min<size_t>((pixels + 255) / 256, 8192), 256, 0, e->stream>>>(
            dn->padded_in, dst, l0.out_mat_stride, dn->pin_ic, dn->pin_ih, dn->pin_iw, dn->pin_ph, dn->pin_pw, dn->pin_pad, pixels);
        e->launches++;
        CUDA_TRY(cudaGetLastError());
    }
    return 0;
}

bool engine_in_service(Engine *e) { return e && e->service; }
int engine_service_tokens(Engine *e, nasm_t *nasm, const int *ids_host) {
    if (!e || !e->service || !ids_host) return -1;
    return svc_attach(e, nasm, nullptr, ids_host, false);
}

int engine_set_tokens(nasm_t *nasm, const int *ids_host) {
    DeviceNasm *dn = nasm->dev;
    if (!dn || !ids_host) return -1;
    Engine *e = dn->e;
    aspen_dnn_t *dnn = nasm->dnn;
    CUDA_TRY(cudaSetDevice(e->device));
    const nasm_ldata_t &l0 = nasm->ldata[0];
    const unsigned M = l0.out_mat_dims[OUT_H];
    const size_t n_tokens = l0.out_mat_dims[OUT_W];
    if (dnn->emb_token.empty() || dnn->emb_width != M || M % 4 != 0 || l0.out_mat_stride % 4 != 0) {
        ASPEN_ERR("token input: the dnn has no embedding table of width %u (aspen_b200_dnn_set_embedding), or the width is not a multiple of 4\n", M);
        return -1;
    }
    if (!dnn->emb_position.empty() && nasm->tr_seq_len > dnn->emb_max_pos) { ASPEN_ERR("token input: sequence length %u exceeds the position table (%u rows)\n", nasm->tr_seq_len, dnn->emb_max_pos); return -1; }
    DeviceDnn *dd = dn->dd;
    if (!dd->emb_token) {
        CUDA_TRY(cudaMalloc(&dd->emb_token, dnn->emb_token.size() * sizeof(float)));
        CUDA_TRY(cudaMemcpy(dd->emb_token, dnn->emb_token.data(), dnn->emb_token.size() * sizeof(float), cudaMemcpyHostToDevice));
        if (!dnn->emb_position.empty()) {
            CUDA_TRY(cudaMalloc(&dd->emb_position, dnn->emb_position.size() * sizeof(float)));
            CUDA_TRY(cudaMemcpy(dd->emb_position, dnn->emb_position.data(), dnn->emb_position.size() * sizeof(float), cudaMemcpyHostToDevice));
        }
    }
    if (!dn->ids_stage) CUDA_TRY(cudaMalloc(&dn->ids_stage, n_tokens * sizeof(int)));
    cudaStream_t io = io_stream(e, nasm);
    dn->res_valid = false;
    // ids by DMA on the transfer stream (after the previous gather has read the staging copy), gather on the compute stream
    CUDA_TRY(cudaStreamWaitEvent(io, dn->in_consumed, 0));
    CUDA_TRY(cudaMemcpyAsync(dn->ids_stage, ids_host, n_tokens * sizeof(int), cudaMemcpyHostToDevice, io));
    CUDA_TRY(cudaStreamSynchronize(io));     // the caller may reuse its buffer as soon as we return
    float *dst = (float *)((char *)dn->arena + dn->ldata_off[0]);
    const size_t work = n_tokens * (M / 4);
    embedding_gather<<<(unsigned)std::min<size_t>((work + 255) / 256, 4096), 256, 0, e->stream>>>(
        dst, l0.out_mat_stride, dn->ids_stage, dd->emb_token, dd->emb_position, M, nasm->tr_seq_len ? nasm->tr_seq_len : 1u, dnn->emb_vocab, n_tokens,
        dn->round_input ? 1 : 0);
    e->launches++;
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaEventRecord(dn->in_consumed, e->stream));
    return 0;
}

int engine_attach_nasm(Engine *e, nasm_t *nasm, const void *input_host) {
    if (!e) return -1;
    if (e->service) return svc_attach(e, nasm, input_host, nullptr, false);
    CUDA_TRY(cudaSetDevice(e->device));
    if (nasm->dev && nasm->dev->e != e) { engine_detach_nasm(nasm); }
    if (!nasm->dev) {
        if (build_device_nasm(e, nasm) != 0) { engine_detach_nasm(nasm); return -1; }
        CUDA_TRY(cudaStreamSynchronize(e->stream));   // the image (zeroed arena, descriptors) is in place before the transfer stream touches it
    }
    if (engine_set_input(nasm, input_host) != 0) return -1;
    nasm->dev->armed = true;
    *nasm->dev->completed_h = 0;
    return 0;
}

void engine_detach_nasm(nasm_t *nasm) {
    DeviceNasm *dn = nasm->dev;
    if (!dn) return;
    Engine *e = dn->e;
    cudaSetDevice(e->device);
    svc_halt(e);
    e->svc_pool.erase(std::remove(e->svc_pool.begin(), e->svc_pool.end(), nasm), e->svc_pool.end());
    if (e->running) { cudaStreamSynchronize(e->stream); e->running = false; }
    e->in_flight.erase(std::remove(e->in_flight.begin(), e->in_flight.end(), nasm), e->in_flight.end());
    e->uploaded.clear();
    free_device_nasm(dn);
    nasm->dev = nullptr;
}

int engine_rearm(Engine *e, nasm_t *nasm) {
    if (!nasm->dev) return -1;
    if (e->service) return svc_attach(e, nasm, nullptr, nullptr, true);
    if (e->running && std::find(e->in_flight.begin(), e->in_flight.end(), nasm) != e->in_flight.end()) {
        // re-arming a graph the device is still draining: let that run finish first
        cudaSetDevice(e->device);
        cudaStreamSynchronize(e->stream);
        e->running = false;
        e->in_flight.clear();
    }
    nasm->dev->armed = true;
    *nasm->dev->completed_h = 0;
    return 0;
}

static int launch_run(Engine *e, const std::vector<nasm_t *> &run) {
    std::vector<NasmDev> images(run.size());
    unsigned total = 0, n_init = 0, n_input = 0;
    for (size_t i = 0; i < run.size(); i++) {
        DeviceNasm *dn = run[i]->dev;
        images[i] = dn->host;
        images[i].tile_base = total;
        images[i].queue_base = n_init;
        total += dn->host.n_tiles;
        n_init += dn->host.n_init;
        n_input += dn->host.n_input_tiles;
    }
    if (run.size() > e->nasms_cap) {
        cudaFree(e->nasms_d);
        e->nasms_d = nullptr;
        e->nasms_cap = 0;
        CUDA_TRY(cudaMalloc(&e->nasms_d, run.size() * sizeof(NasmDev)));
        e->nasms_cap = (unsigned)run.size();
    }
    if (total > e->queue_cap) {
        cudaFree(e->queue);
        e->queue = nullptr;
        e->queue_cap = 0;
        CUDA_TRY(cudaMalloc(&e->queue, (size_t)total * sizeof(unsigned)));
        e->queue_cap = total;
    }
    if (run != e->uploaded) {
        // cudaMemcpyAsync from pageable memory returns after the source has been staged
        CUDA_TRY(cudaMemcpyAsync(e->nasms_d, images.data(), images.size() * sizeof(NasmDev), cudaMemcpyHostToDevice, e->stream));
        unsigned n_nasm = (unsigned)run.size();
        CUDA_TRY(cudaMemcpyAsync(&e->ctrl->n_nasm, &n_nasm, sizeof(unsigned), cudaMemcpyHostToDevice, e->stream));
        e->uploaded = run;
    }
    e->status_h->status = 0;
    e->status_h->tiles_done = 0;
    unsigned arm_blocks = std::min<unsigned>((total + 255) / 256, 1024);
    sched::arm_kernel<<<arm_blocks, 256, 0, e->stream>>>(e->nasms_d, e->ctrl, e->queue, total, n_init, n_input, e->stall_ns, e->pipe_ns, e->run_ahead);
    sched::seed_kernel<<<std::max(1u, std::min<unsigned>((n_init + 255) / 256, 256)), 256, 0, e->stream>>>(e->nasms_d, e->ctrl, e->queue);
    bool any_attention = false;
    for (nasm_t *nasm : run) any_attention |= nasm->dev->fused_attention;
    if (e->precision == 0 && any_attention)
        sched::scheduler_kernel<true, true><<<e->n_ctas, sched::SCHED_THREADS, e->smem_bytes, e->stream>>>(e->nasms_d, e->ctrl, e->queue, e->status_d, e->prof);
    else if (e->precision == 0)
        sched::scheduler_kernel<true><<<e->n_ctas, sched::SCHED_THREADS, e->smem_bytes, e->stream>>>(e->nasms_d, e->ctrl, e->queue, e->status_d, e->prof);
    else
        sched::scheduler_kernel<false><<<e->n_ctas, sched::SCHED_THREADS, e->smem_bytes, e->stream>>>(e->nasms_d, e->ctrl, e->queue, e->status_d, e->prof);
    e->launches += 3;
    CUDA_TRY(cudaGetLastError());
    for (nasm_t *nasm : run) {
        DeviceNasm *dn = nasm->dev;
        if (dn->res_packed) {
            const unsigned last = nasm->num_ldata - 1;
            const nasm_ldata_t &ld = nasm->ldata[last];
            const size_t n = (size_t)ld.out_mat_dims[OUT_H] * ld.out_mat_dims[OUT_W];
            const unsigned blocks = (unsigned)std::min<size_t>((n + XFER_THREADS - 1) / XFER_THREADS, 16384);
            pack_columns<<<blocks, XFER_THREADS, 0, e->stream>>>(dn->res_packed, (const float *)((char *)dn->arena + dn->ldata_off[last]),
                                                                ld.out_mat_dims[OUT_H], ld.out_mat_stride, n);
            e->launches++;
        }
        CUDA_TRY(cudaEventRecord(dn->res_ready, e->stream));
        dn->res_valid = true;
    }
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int engine_run(Engine *e, const std::vector<nasm_t *> &nasms) {
    if (!e) return -1;
    CUDA_TRY(cudaSetDevice(e->device));
    if (e->service) return svc_run(e, nasms);
    std::vector<nasm_t *> run;
    for (nasm_t *n : nasms)
        if (n->dev && n->dev->e == e && n->dev->armed) run.push_back(n);
    if (run.empty()) return 0;
    if (e->running) {   // one persistent kernel at a time per group: the armed graphs join the next launch
        CUDA_TRY(cudaStreamSynchronize(e->stream));
        e->running = false;
        e->in_flight.clear();
    }
    if (launch_run(e, run) != 0) return -1;
    for (nasm_t *n : run) { n->dev->armed = false; n->dev->ran = true; }
    e->in_flight = run;
    e->running = true;
    return 0;
}

int engine_stop(Engine *e) {
    if (e && e->service) { CUDA_TRY(cudaSetDevice(e->device)); return svc_halt(e); }
    if (!e || !e->running) return 0;
    CUDA_TRY(cudaSetDevice(e->device));
    if (cudaStreamQuery(e->stream) == cudaErrorNotReady) {
        // cooperative stop: CTAs leave after their current tile (ref src/dse.c:215-232)
        unsigned one = 1;
        cudaMemcpyAsync(&e->ctrl->stop, &one, sizeof(unsigned), cudaMemcpyHostToDevice, e->side);
    }
    cudaError_t err = cudaStreamSynchronize(e->stream);
    // the stop write itself must have landed (or been dropped by a kernel that had already left) before the next arm
    // kernel clears the flag: a write that arrived after it would end the next run after its first tiles
    cudaStreamSynchronize(e->side);
    e->running = false;
    for (nasm_t *n : e->in_flight)
        if (n->dev && *(volatile unsigned *)n->dev->completed_h == 0) n->dev->armed = true;   // unfinished: restarts at the next run
    e->in_flight.clear();
    if (err != cudaSuccess) { ASPEN_ERR("CUDA error after run: %s\n", cudaGetErrorString(err)); e->status_h->status = ASPEN_B200_ERR_CUDA; return -1; }
    return 0;
}

unsigned int engine_poll_nasm(nasm_t *nasm) {
    if (nasm->dev && nasm->dev->e->service) return svc_done(nasm->dev) ? 1u : 0u;
    return nasm->dev ? *(volatile unsigned *)nasm->dev->completed_h : 0;
}

int engine_wait_nasm(nasm_t *nasm) {
    DeviceNasm *dn = nasm->dev;
    if (!dn) return -1;
    Engine *e = dn->e;
    cudaSetDevice(e->device);
    if (e->service) return svc_wait(nasm);
    for (unsigned spin = 0;; spin++) {
        if (*(volatile unsigned *)dn->completed_h) return 0;
        if (!e->running) return -1;
        cudaError_t q = cudaStreamQuery(e->stream);
        if (q == cudaSuccess) return *(volatile unsigned *)dn->completed_h ? 0 : -1;   // kernel left without finishing this graph
        if (q != cudaErrorNotReady) { ASPEN_ERR("CUDA error while waiting: %s\n", cudaGetErrorString(q)); e->status_h->status = ASPEN_B200_ERR_CUDA; return -1; }
        if (spin > 64) sched_yield();
    }
}

long engine_read_ldata(nasm_t *nasm, unsigned int idx, float *out) {
    DeviceNasm *dn = nasm->dev;
    if (!dn) return -1;
    Engine *e = dn->e;
    if (cudaSetDevice(e->device) != cudaSuccess) return -1;
    const nasm_ldata_t &ld = nasm->ldata[idx];
    const size_t n = (size_t)ld.out_mat_dims[OUT_H] * ld.out_mat_dims[OUT_W];
    const float *src = (const float *)((char *)dn->arena + dn->ldata_off[idx]);
    if (e->service && e->svc_live) {
        // a kernel could not start next to the resident one: strided matrices are packed by the copy engine
        const size_t row = (size_t)ld.out_mat_dims[OUT_H] * sizeof(float);
        if (cudaMemcpy2DAsync(out, row, src, (size_t)ld.out_mat_stride * sizeof(float), row, ld.out_mat_dims[OUT_W], cudaMemcpyDeviceToHost, e->io) != cudaSuccess ||
            cudaStreamSynchronize(e->io) != cudaSuccess) {
            ASPEN_ERR("CUDA error reading layer %u: %s\n", idx, cudaGetErrorString(cudaGetLastError()));
            return -1;
        }
        return (long)n;
    }
    if (idx == nasm->num_ldata - 1 && dn->res_valid) {
        // the last layer of a graph that has run: already gathered (or packed by layout); DMA only
        if (cudaStreamWaitEvent(e->io, dn->res_ready, 0) != cudaSuccess) return -1;
        if (cudaMemcpyAsync(out, dn->res_packed ? dn->res_packed : src, n * sizeof(float), cudaMemcpyDeviceToHost, e->io) != cudaSuccess) return -1;
        if (cudaStreamSynchronize(e->io) != cudaSuccess) { ASPEN_ERR("CUDA error reading layer %u: %s\n", idx, cudaGetErrorString(cudaGetLastError())); return -1; }
        return (long)n;
    }
    cudaStream_t st = io_stream(e, nasm);
    if (ld.out_mat_stride == ld.out_mat_dims[OUT_H]) {
        if (cudaMemcpyAsync(out, src, n * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
    } else {
        if (ensure_xfer(e, n * sizeof(float)) != 0) return -1;
        unsigned blocks = (unsigned)std::min<size_t>((n + XFER_THREADS - 1) / XFER_THREADS, 16384);
        pack_columns<<<blocks, XFER_THREADS, 0, st>>>(e->xfer, src, ld.out_mat_dims[OUT_H], ld.out_mat_stride, n);
        e->launches++;
        if (cudaMemcpyAsync(out, e->xfer, n * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
    }
    if (cudaStreamSynchronize(st) != cudaSuccess) { ASPEN_ERR("CUDA error reading layer %u: %s\n", idx, cudaGetErrorString(cudaGetLastError())); return -1; }
    return (long)n;
}

double engine_time_runs(Engine *e, const std::vector<nasm_t *> &nasms, unsigned int warmup, unsigned int iters, unsigned long long *launches) {
    if (!e) return -1.0;
    if (cudaSetDevice(e->device) != cudaSuccess) return -1.0;
    cudaEvent_t t0, t1;
    if (cudaEventCreate(&t0) != cudaSuccess || cudaEventCreate(&t1) != cudaSuccess) return -1.0;
    unsigned long long l0 = 0;
    std::vector<nasm_t *> run;
    for (nasm_t *n : nasms)
        if (n->dev && n->dev->e == e) run.push_back(n);
    if (run.empty()) return -1.0;
    if (svc_halt(e) != 0) return -1.0;
    if (e->running) { cudaStreamSynchronize(e->stream); e->running = false; e->in_flight.clear(); }
    for (unsigned i = 0; i < warmup + iters; i++) {
        if (i == warmup) { cudaEventRecord(t0, e->stream); l0 = e->launches; }
        if (launch_run(e, run) != 0) return -1.0;   // back to back on one stream: arming waits for the previous run
    }
    cudaEventRecord(t1, e->stream);
    cudaError_t err = cudaStreamSynchronize(e->stream);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, t0, t1);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    for (nasm_t *n : run) { n->dev->armed = false; n->dev->ran = true; }
    if (launches) *launches = e->launches - l0;
    if (err != cudaSuccess || e->status_h->status != 0) {
        ASPEN_ERR("timed runs failed: cuda=%s engine status=%u (info %u %u)\n", cudaGetErrorString(err), e->status_h->status, e->status_h->info0, e->status_h->info1);
        return -1.0;
    }
    for (nasm_t *n : run)
        if (*(volatile unsigned *)n->dev->completed_h == 0) { ASPEN_ERR("timed runs: a graph did not complete\n"); return -1.0; }
    return (double)ms;
}

// ---- service mode ---------------------------------------------------------------------------------------------------
// Host side of the resident kernel described in scheduler.cuh.  dse_group_run launches it over every graph of the pool;
// rpool_add_nasm* on a graph it serves uploads the input on the transfer stream and then writes the graph's pass number
// to the device with a 4-byte copy on the same stream; dse_wait_for_nasm_completion polls the graph's mapped word;
// dse_group_stop asks the kernel to leave and waits for it.  The kernel also leaves by itself (idle, or the queue of
// the launch used up); whoever next runs or waits launches it again when passes are still owed, and a pass cut short
// simply starts over (a pass only reads its input and writes its own matrices).
// Nothing that allocates or frees device memory, and no kernel, may be issued while the kernel is resident: those paths
// stop it first.
static bool svc_done(const DeviceNasm *dn) { return *(volatile unsigned *)dn->svc_done_h == dn->svc_armed; }

static int svc_halt(Engine *e) {
    if (!e->svc_live) return 0;
    if (cudaStreamQuery(e->stream) == cudaErrorNotReady) {
        unsigned one = 1;
        cudaMemcpyAsync(&e->ctrl->svc_stop, &one, sizeof(unsigned), cudaMemcpyHostToDevice, e->side);
    }
    cudaError_t err = cudaStreamSynchronize(e->stream);
    cudaStreamSynchronize(e->side);
    cudaStreamSynchronize(e->io);
    e->svc_live = false;
    e->svc_graphs.clear();
    if (err != cudaSuccess) { ASPEN_ERR("CUDA error after a service run: %s\n", cudaGetErrorString(err)); e->status_h->status = ASPEN_B200_ERR_CUDA; return -1; }
    return 0;
}

static int svc_launch(Engine *e, const std::vector<nasm_t *> &graphs, unsigned stop_when_done) {
    std::vector<NasmDev> images(graphs.size());
    unsigned total = 0;
    for (size_t i = 0; i < graphs.size(); i++) {
        nasm_t *nasm = graphs[i];
        DeviceNasm *dn = nasm->dev;
        if (dn->fused_attention) { ASPEN_ERR("service mode: graphs with the fused attention tile are run per launch only\n"); return -1; }
        NasmDev &G = images[i];
        G = dn->host;
        G.tile_base = total;
        total += G.n_tiles;
        G.svc = dn->svc_d; G.svc_base = *(volatile unsigned *)dn->svc_done_h; G.completed = dn->svc_done_d;
        G.n_exec = dn->n_exec; G.n_input = dn->n_input;
        InputDev &I = G.input;
        memset(&I, 0, sizeof I);
        I.round = dn->round_input ? 1u : 0u;
        if (dn->svc_ids) {
            I.ids = dn->ids_stage; I.emb_tok = dn->dd->emb_token; I.emb_pos = dn->dd->emb_position;
            I.emb_vocab = nasm->dnn->emb_vocab; I.emb_seq = nasm->tr_seq_len ? nasm->tr_seq_len : 1u;
        } else I.stage = dn->in_stage;
        I.padded = dn->padded_in; I.IC = dn->pin_ic; I.IH = dn->pin_ih; I.IW = dn->pin_iw; I.PH = dn->pin_ph; I.PW = dn->pin_pw; I.pad = dn->pin_pad;
    }
    if (total >= (1u << 30)) { ASPEN_ERR("service mode: too many tiles\n"); return -1; }
    // queue of the launch: room for a number of passes; when it is used up the kernel leaves and is launched again
    const unsigned passes = std::max(4u, std::min(256u, (8u << 20) / std::max(total, 1u)));
    const unsigned cap = total * passes;
    if (graphs.size() > e->nasms_cap) {
        cudaFree(e->nasms_d);
        e->nasms_d = nullptr;
        e->nasms_cap = 0;
        CUDA_TRY(cudaMalloc(&e->nasms_d, graphs.size() * sizeof(NasmDev)));
        e->nasms_cap = (unsigned)graphs.size();
    }
    if (cap > e->queue_cap) {
        cudaFree(e->queue);
        e->queue = nullptr;
        e->queue_cap = 0;
        CUDA_TRY(cudaMalloc(&e->queue, (size_t)cap * sizeof(unsigned)));
        e->queue_cap = cap;
    }
    e->uploaded.clear();     // the per-launch path must upload its own images again
    CUDA_TRY(cudaMemcpyAsync(e->nasms_d, images.data(), images.size() * sizeof(NasmDev), cudaMemcpyHostToDevice, e->stream));
    unsigned n_nasm = (unsigned)graphs.size();
    CUDA_TRY(cudaMemcpyAsync(&e->ctrl->n_nasm, &n_nasm, sizeof(unsigned), cudaMemcpyHostToDevice, e->stream));
    for (nasm_t *nasm : graphs)
        CUDA_TRY(cudaMemcpyAsync(&nasm->dev->svc_d[SVC_TARGET], &nasm->dev->svc_armed, sizeof(unsigned), cudaMemcpyHostToDevice, e->stream));
    // pass numbers written later (transfer stream) must not be overtaken by the ones above
    CUDA_TRY(cudaEventRecord(e->svc_armed_ev, e->stream));
    CUDA_TRY(cudaStreamWaitEvent(e->io, e->svc_armed_ev, 0));
    e->status_h->status = 0;
    e->status_h->tiles_done = 0;
    sched::svc_arm_kernel<<<std::min<unsigned>((cap + 255) / 256, 2048), 256, 0, e->stream>>>(e->nasms_d, e->ctrl, e->queue, cap, total, e->stall_ns, e->pipe_ns,
                                                                                               e->idle_ns, stop_when_done, e->svc_ahead);
    if (e->precision == 0)
        sched::scheduler_kernel<true, false, true><<<e->n_ctas, sched::SCHED_THREADS, e->smem_bytes, e->stream>>>(e->nasms_d, e->ctrl, e->queue, e->status_d, e->prof);
    else
        sched::scheduler_kernel<false, false, true><<<e->n_ctas, sched::SCHED_THREADS, e->smem_bytes, e->stream>>>(e->nasms_d, e->ctrl, e->queue, e->status_d, e->prof);
    e->launches += 2;
    CUDA_TRY(cudaGetLastError());
    e->svc_graphs = graphs;
    e->svc_live = true;
    for (nasm_t *nasm : graphs) { nasm->dev->ran = true; nasm->dev->res_valid = false; }
    return 0;
}

static void svc_pool_add(Engine *e, const std::vector<nasm_t *> &nasms) {
    for (nasm_t *n : nasms)
        if (n->dev && n->dev->e == e && std::find(e->svc_pool.begin(), e->svc_pool.end(), n) == e->svc_pool.end()) e->svc_pool.push_back(n);
}
static bool svc_serves(Engine *e, const nasm_t *nasm) {
    return e->svc_live && std::find(e->svc_graphs.begin(), e->svc_graphs.end(), nasm) != e->svc_graphs.end();
}

// dse_group_run in service mode.
static int svc_run(Engine *e, const std::vector<nasm_t *> &nasms) {
    svc_pool_add(e, nasms);
    const std::vector<nasm_t *> graphs = e->svc_pool;
    if (graphs.empty()) return 0;
    if (e->svc_live) {
        bool served = cudaStreamQuery(e->stream) == cudaErrorNotReady;
        for (nasm_t *n : graphs) served = served && svc_serves(e, n);
        if (served) return 0;         // the passes asked for since were signalled to the resident kernel
        if (svc_halt(e) != 0) return -1;
    }
    bool owed = false;
    for (nasm_t *n : graphs) owed = owed || !svc_done(n->dev);
    return owed ? svc_launch(e, graphs, 0u) : 0;
}

// dse_wait_for_nasm_completion in service mode.
static int svc_wait(nasm_t *nasm) {
    DeviceNasm *dn = nasm->dev;
    Engine *e = dn->e;
    unsigned relaunches = 0;
    for (unsigned spin = 0;; spin++) {
        if (svc_done(dn)) return 0;
        if (e->status_h->status != 0) return -1;
        cudaError_t q = svc_serves(e, nasm) ? cudaStreamQuery(e->stream) : cudaSuccess;
        if (q == cudaSuccess) {
            // no kernel serves the graph (never launched for it; or it left: idle, queue used up, a request that just
            // missed it): launch for everything that is owed.  Every launch completes at least the pass it was launched
            // for unless it reports an error, so a few launches in a row without this graph completing is a fault.
            if (svc_done(dn)) return 0;
            if (e->status_h->status != 0 || ++relaunches > 1000u) { ASPEN_ERR("service mode: the graph's pass does not complete\n"); return -1; }
            if (svc_halt(e) != 0 || svc_launch(e, e->svc_pool, 0u) != 0) return -1;
        } else if (q != cudaErrorNotReady) {
            ASPEN_ERR("CUDA error while waiting: %s\n", cudaGetErrorString(q));
            e->status_h->status = ASPEN_B200_ERR_CUDA;
            return -1;
        }
        if (spin > 64) sched_yield();
    }
}

// rpool_add_nasm* in service mode: upload (input_host, or ids_host, or neither = keep what layer 0 / the staging copy
// holds) and ask for one more pass of the graph.
static int svc_attach(Engine *e, nasm_t *nasm, const void *input_host, const int *ids_host, bool keep_input) {
    CUDA_TRY(cudaSetDevice(e->device));
    if (nasm->dev && nasm->dev->e != e) { if (svc_halt(e) != 0) return -1; engine_detach_nasm(nasm); }
    if (!nasm->dev) {
        if (svc_halt(e) != 0) return -1;
        if (build_device_nasm(e, nasm) != 0) { engine_detach_nasm(nasm); return -1; }
        CUDA_TRY(cudaStreamSynchronize(e->stream));
    }
    DeviceNasm *dn = nasm->dev;
    svc_pool_add(e, std::vector<nasm_t *>{nasm});
    // the previous pass of this graph is still owed: its input must stay until that pass is complete
    if (!svc_done(dn) && svc_wait(nasm) != 0) return -1;
    const nasm_ldata_t &l0 = nasm->ldata[0];
    const size_t n = (size_t)l0.out_mat_dims[OUT_H] * l0.out_mat_dims[OUT_W];
    float *dst = (float *)((char *)dn->arena + dn->ldata_off[0]);
    if (ids_host) {
        aspen_dnn_t *dnn = nasm->dnn;
        const unsigned M = l0.out_mat_dims[OUT_H];
        if (dnn->emb_token.empty() || dnn->emb_width != M || M % 4 != 0 || l0.out_mat_stride % 4 != 0 || l0.ninst_tile_dims[OUT_H] % 4 != 0) {
            ASPEN_ERR("token input: the dnn has no embedding table of width %u (aspen_b200_dnn_set_embedding), or the width is not a multiple of 4\n", M);
            return -1;
        }
        if (!dnn->emb_position.empty() && nasm->tr_seq_len > dnn->emb_max_pos) { ASPEN_ERR("token input: sequence length %u exceeds the position table (%u rows)\n", nasm->tr_seq_len, dnn->emb_max_pos); return -1; }
        DeviceDnn *dd = dn->dd;
        if (!dd->emb_token || !dn->ids_stage || !dn->svc_ids) {
            if (svc_halt(e) != 0) return -1;          // allocations, and the graph's image changes
            if (!dd->emb_token) {
                CUDA_TRY(cudaMalloc(&dd->emb_token, dnn->emb_token.size() * sizeof(float)));
                CUDA_TRY(cudaMemcpy(dd->emb_token, dnn->emb_token.data(), dnn->emb_token.size() * sizeof(float), cudaMemcpyHostToDevice));
                if (!dnn->emb_position.empty()) {
                    CUDA_TRY(cudaMalloc(&dd->emb_position, dnn->emb_position.size() * sizeof(float)));
                    CUDA_TRY(cudaMemcpy(dd->emb_position, dnn->emb_position.data(), dnn->emb_position.size() * sizeof(float), cudaMemcpyHostToDevice));
                }
            }
            if (!dn->ids_stage) CUDA_TRY(cudaMalloc(&dn->ids_stage, (size_t)l0.out_mat_dims[OUT_W] * sizeof(int)));
            dn->svc_ids = true;
        }
        CUDA_TRY(cudaMemcpyAsync(dn->ids_stage, ids_host, (size_t)l0.out_mat_dims[OUT_W] * sizeof(int), cudaMemcpyHostToDevice, e->io));
        CUDA_TRY(cudaStreamSynchronize(e->io));       // the caller may reuse its buffer as soon as we return
    } else if (!keep_input) {
        if (dn->svc_ids) { if (svc_halt(e) != 0) return -1; dn->svc_ids = false; }
        if (!input_host) {
            // no input: the staging copy (or layer 0) is cleared; a memset may be a kernel, so the resident kernel leaves first
            if (svc_halt(e) != 0) return -1;
            CUDA_TRY(cudaMemsetAsync(dn->in_stage ? dn->in_stage : dst, 0, dn->in_stage ? n * sizeof(float) : l0.out_mat_mem_size, e->stream));
            CUDA_TRY(cudaStreamSynchronize(e->stream));
        } else {
            CUDA_TRY(cudaMemcpyAsync(dn->in_stage ? dn->in_stage : dst, input_host, n * sizeof(float), cudaMemcpyHostToDevice, e->io));
            CUDA_TRY(cudaStreamSynchronize(e->io));
        }
    }
    dn->svc_armed++;
    dn->res_valid = false;
    if (svc_serves(e, nasm))
        CUDA_TRY(cudaMemcpyAsync(&dn->svc_d[SVC_TARGET], &dn->svc_armed, sizeof(unsigned), cudaMemcpyHostToDevice, e->io));
    return 0;
}

int engine_set_service(Engine *e, int on) {
    if (!e) return -1;
    CUDA_TRY(cudaSetDevice(e->device));
    if (e->service == (on != 0)) return 0;
    if (e->service) { if (svc_halt(e) != 0) return -1; e->svc_pool.clear(); }
    else if (e->running) { cudaStreamSynchronize(e->stream); e->running = false; e->in_flight.clear(); }
    e->service = on != 0;
    return 0;
}

// `passes` passes, dealt round robin to the pool's graphs, inside service launches that leave when they are done;
// device time between CUDA events on the compute stream.  Inputs are whatever the graphs hold (layer 0 / staging copy).
double engine_time_passes(Engine *e, const std::vector<nasm_t *> &nasms, unsigned int warmup, unsigned int passes, unsigned long long *launches) {
    if (!e || !e->service) return -1.0;
    if (cudaSetDevice(e->device) != cudaSuccess || svc_halt(e) != 0) return -1.0;
    svc_pool_add(e, nasms);
    const std::vector<nasm_t *> graphs = e->svc_pool;
    if (graphs.empty()) return -1.0;
    cudaEvent_t t0, t1;
    if (cudaEventCreate(&t0) != cudaSuccess || cudaEventCreate(&t1) != cudaSuccess) return -1.0;
    float ms = 0.f;
    unsigned long long l0 = 0;
    for (int phase = 0; phase < 2; phase++) {
        const unsigned count = phase == 0 ? warmup : passes;
        if (count == 0) continue;
        for (size_t i = 0; i < graphs.size(); i++)
            graphs[i]->dev->svc_armed += count / (unsigned)graphs.size() + (i < count % graphs.size() ? 1u : 0u);
        if (phase == 1) { cudaEventRecord(t0, e->stream); l0 = e->launches; }
        for (unsigned tries = 0;; tries++) {
            if (svc_launch(e, graphs, 1u) != 0) return -1.0;
            if (phase == 1) cudaEventRecord(t1, e->stream);
            if (svc_halt(e) != 0 || e->status_h->status != 0) {
                ASPEN_ERR("timed passes failed: engine status %u (info %u %u)\n", e->status_h->status, e->status_h->info0, e->status_h->info1);
                return -1.0;
            }
            bool done = true;
            for (nasm_t *n : graphs) done = done && svc_done(n->dev);
            if (done) break;
            if (tries > 100000u) return -1.0;      // each launch completes at least one pass or reports a stall
        }
    }
    cudaEventElapsedTime(&ms, t0, t1);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    if (launches) *launches = e->launches - l0;
    return (double)ms;
}

void engine_flush() {}

// Sums the per-CTA time accounting (ASPEN_B200_PROFILE=1) into out[PROF_SLOTS] and clears it.
int engine_read_profile(Engine *e, unsigned long long *out, unsigned *n_ctas) {
    if (!e || !e->prof) return -1;
    CUDA_TRY(cudaSetDevice(e->device));
    if (svc_halt(e) != 0) return -1;
    CUDA_TRY(cudaStreamSynchronize(e->stream));
    std::vector<unsigned long long> h((size_t)e->n_ctas * sched::PROF_SLOTS);
    CUDA_TRY(cudaMemcpy(h.data(), e->prof, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    CUDA_TRY(cudaMemset(e->prof, 0, h.size() * sizeof(unsigned long long)));
    for (unsigned s = 0; s < sched::PROF_SLOTS; s++) out[s] = 0;
    for (unsigned c = 0; c < e->n_ctas; c++)
        for (unsigned s = 0; s < sched::PROF_SLOTS; s++) out[s] += h[(size_t)c * sched::PROF_SLOTS + s];
    if (n_ctas) *n_ctas = e->n_ctas;
    return 0;
}
