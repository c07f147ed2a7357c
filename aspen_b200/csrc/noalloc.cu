// aspen_b200_matmul_noalloc: one matmul layer run as a tile graph by the persistent scheduler
// kernel, for callers that must not allocate.
//
// Who cannot allocate: plug-ins that are handed a fixed memory budget by their host framework (a
// serving runtime that pre-sizes every pool at start-up and treats a later cudaMalloc as a bug), and
// latency-critical loops where the implicit device synchronisation of cudaMalloc / cudaFree is not
// acceptable.  The regular API builds a device image per nasm (arena, descriptors, counters, queue)
// with cudaMalloc; this entry point keeps everything the scheduler needs besides the caller's own
// input / weight / output buffers in one file-scope device array of fixed size.
//
// Consequences of the fixed array, all documented in the header too:
//   * sizes are limited (NOALLOC_MAX_TILES output tiles of 128 x 128); larger calls are rejected;
//   * every call on a device uses the same array: it keeps the previous call's contents, so the
//     set-up kernel rewrites all of it that a run reads (counters and queue start from zero again);
//     two calls that overlap on the GPU (different streams, or different host threads) race;
//   * the first call on a device looks the array's address up (cudaGetSymbolAddress) -- make that
//     call before any stream capture;
//   * every call ends by reading the scheduler's status back and synchronising its stream.
#include "internal.h"
#include "scheduler.cuh"

#include <cuda_runtime.h>
#include <algorithm>

namespace {

constexpr unsigned NOALLOC_MAX_TILES = ASPEN_B200_NOALLOC_MAX_TILES;
constexpr unsigned NOALLOC_TILE = 128;

struct NoAllocScratch {
    CtrlDev ctrl;
    StatusHost status;
    NasmDev nasm;
    LayerDev layer;
    unsigned layer_done, layer_tiles, layers_completed, completed;
    unsigned queue[NOALLOC_MAX_TILES];
    unsigned dep[NOALLOC_MAX_TILES];
    TileDev tiles[NOALLOC_MAX_TILES];
};

// The scratch memory itself.  In host code this name is only a handle for cudaGetSymbolAddress, never
// a pointer a kernel could use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

struct NoAllocArgs {
    const float *x, *w, *bias;
    float *out;
    unsigned n_cols, k, m;
    int act;
    unsigned long long stall_ns, pipe_ns;
};

// Rebuilds the whole image in the scratch array: descriptors, zeroed counters, a queue that already
// holds every tile (a single layer has no dependencies between its tiles).
__global__ void noalloc_setup(NoAllocScratch *s, NoAllocArgs a) {
    const unsigned tiles_h = (a.m + NOALLOC_TILE - 1) / NOALLOC_TILE, tiles_w = (a.n_cols + NOALLOC_TILE - 1) / NOALLOC_TILE;
    const unsigned n = tiles_h * tiles_w;
    const unsigned stride = gridDim.x * blockDim.x, t0 = blockIdx.x * blockDim.x + threadIdx.x;
    for (unsigned t = t0; t < n; t += stride) {
        TileDev T;
        T.layer = 0;
        T.pos_h = (t % tiles_h) * NOALLOC_TILE;
        T.pos_w = (t / tiles_h) * NOALLOC_TILE;
        T.tile_h = min(NOALLOC_TILE, a.m - T.pos_h);
        T.tile_w = min(NOALLOC_TILE, a.n_cols - T.pos_w);
        T.child_off = 0; T.child_cnt = 0; T.need = 0; T.flags = 0;
        s->tiles[t] = T;
        s->queue[t] = t + 1u;
        s->dep[t] = 0u;
    }
    if (t0 != 0) return;
    LayerDev L;
    memset(&L, 0, sizeof L);
    L.type = MATMUL_LAYER; L.act = a.act;
    L.out = a.out; L.ldc = a.m; L.H = a.m; L.W = a.n_cols;
    L.in0 = a.x; L.ld0 = a.k; L.H0 = a.k;
    L.weight = a.w; L.bias = a.bias;
    L.K = a.k; L.Kpad = a.k; L.rows = a.m;
    L.wmap = -1; L.amap = -1; L.resmap = -1; L.bw = 128;
    L.a_vec4 = (a.k % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.w)) % 16 == 0);
    s->layer = L;
    NasmDev G;
    memset(&G, 0, sizeof G);
    G.layers = &s->layer; G.tiles = s->tiles; G.children = s->dep; G.dep = s->dep; G.dep_init = s->dep;
    G.layer_done = &s->layer_done; G.layer_tiles = &s->layer_tiles; G.init_ready = s->queue;
    G.layers_completed = &s->layers_completed; G.completed = &s->completed;
    G.n_tiles = n; G.n_layers = 1; G.n_init = n;
    s->nasm = G;
    s->layer_done = 0; s->layer_tiles = n; s->layers_completed = 0; s->completed = 0;
    s->status.status = 0; s->status.info0 = 0; s->status.info1 = 0; s->status.tiles_done = 0;
    CtrlDev c;
    memset(&c, 0, sizeof c);
    c.head = 0; c.tail = n; c.done = 0; c.total = n; c.cap = n; c.n_nasm = 1;
    c.stall_ns = a.stall_ns; c.pipe_ns = a.pipe_ns;
    s->ctrl = c;
}

NoAllocScratch *g_scratch_ptr[16] = {};
size_t g_smem_bytes = sizeof(tc::Shared) + 1024;

}  // namespace

extern "C" int aspen_b200_matmul_noalloc(const float *x_dev, const float *w_dev, const float *bias_dev, float *out_dev,
                                         unsigned int n_cols, unsigned int k, unsigned int m, int activation, void *cuda_stream) {
    if (!x_dev || !w_dev || !out_dev || n_cols == 0 || k == 0 || m == 0) {
        ASPEN_ERR("aspen_b200_matmul_noalloc: NULL buffer or empty shape\n");
        return -1;
    }
    if (activation < 0 || activation >= NUM_ACTIVATIONS) { ASPEN_ERR("aspen_b200_matmul_noalloc: unknown activation %d\n", activation); return -1; }
    // 64-bit: m or n_cols close to 2^32 must not wrap into a small tile count
    const unsigned long long tiles = (((unsigned long long)m + NOALLOC_TILE - 1) / NOALLOC_TILE) * (((unsigned long long)n_cols + NOALLOC_TILE - 1) / NOALLOC_TILE);
    if (tiles > NOALLOC_MAX_TILES) {
        ASPEN_ERR("aspen_b200_matmul_noalloc: %u x %u outputs need %llu tiles of 128 x 128; the fixed scratch array holds %u. "
                  "Use the regular API (it allocates) for larger layers.\n", m, n_cols, tiles, NOALLOC_MAX_TILES);
        return -2;
    }
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= 16) { ASPEN_ERR("aspen_b200_matmul_noalloc: no current CUDA device (%s)\n", cudaGetErrorString(err)); return -3; }
    if (!g_scratch_ptr[dev]) {
        // once per device, with that device current: the device address behind the symbol
        void *p = nullptr;
        err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (err != cudaSuccess || !p) { ASPEN_ERR("aspen_b200_matmul_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(err)); return -3; }
        g_scratch_ptr[dev] = static_cast<NoAllocScratch *>(p);
    }
    NoAllocScratch *s = g_scratch_ptr[dev];
    int sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess || sms <= 0) { ASPEN_ERR("aspen_b200_matmul_noalloc: cannot query the device (%s)\n", cudaGetErrorString(err)); return -3; }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    NoAllocArgs a{x_dev, w_dev, bias_dev, out_dev, n_cols, k, m, activation, 2000000000ull, 1000000000ull};
    noalloc_setup<<<(unsigned)((tiles + 255) / 256), 256, 0, stream>>>(s, a);
    const unsigned ctas = (unsigned)std::min<unsigned long long>(tiles, (unsigned long long)sms);
    sched::scheduler_kernel<false><<<ctas, sched::SCHED_THREADS, g_smem_bytes, stream>>>(&s->nasm, &s->ctrl, s->queue, &s->status, nullptr);
    err = cudaGetLastError();
    if (err != cudaSuccess) { ASPEN_ERR("aspen_b200_matmul_noalloc: launch failed: %s\n", cudaGetErrorString(err)); return -3; }
    // synchronous: the status word lives in the scratch array and the next call overwrites it
    unsigned status[2] = {0, 0};
    err = cudaMemcpyAsync(&status[0], const_cast<const unsigned *>(&s->status.status), sizeof(unsigned), cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess) err = cudaMemcpyAsync(&status[1], &s->completed, sizeof(unsigned), cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) { ASPEN_ERR("aspen_b200_matmul_noalloc: %s\n", cudaGetErrorString(err)); return -3; }
    if (status[0] != 0 || status[1] != 1) { ASPEN_ERR("aspen_b200_matmul_noalloc: scheduler status %u, completed %u\n", status[0], status[1]); return -4; }
    return 0;
}
