// Contraction tiles on the 5th-generation tensor cores (sm_100a): conv, matmul, connected,
// K-attention and V-attention ninst tiles as TF32 tcgen05.mma with fp32 accumulators in TMEM.
//
// Orientation.  A ninst tile is out[column n][row m] (n: pixels / tokens, m: channels / keys /
// features, m contiguous in memory).  The MMA is issued as D[128 x N] with
//     MMA-M (128 TMEM lanes)  <- 128 consecutive tile columns n   (operand "X": activations)
//     MMA-N (<=256 TMEM cols) <- tile rows m                      (operand "W": weights / keys / V)
// so each epilogue thread owns one output column n and writes runs of contiguous m, and the
// K-attention softmax (a reduction over m) stays inside one thread.
//
// Staging.  Both operands are K-major, 32 fp32 (128 bytes) per row and k-chunk, in the 128-byte
// swizzled shared-memory layout UMMA descriptors and TMA share:
//     byte(row r, 16-byte piece c) = r * 128 + ((c ^ (r & 7)) << 4),   stage base 1024-byte aligned.
// Weights arrive by TMA (64-row boxes) straight from the [rows][Kpad] device copy.  Activations arrive
// by TMA wherever the access pattern is a box of the parent matrix -- plain 2-D boxes, a shifted box
// with a zero fix-up of the rows whose tap leaves the image, strided 3-D / 4-D boxes for the stem and the
// stride-2 layers (the table before `enum { A_GATHER ...` lists the kinds) -- and only otherwise are
// gathered by the worker threads with cp.async (zero-fill for padding taps and k >= K).  None of
// them materialises an im2col matrix: a conv tile reads pixel (b, oh*s+kh-p, ow*s+kw-p) of the NHWC
// parent directly.  cp.async writes go through the generic proxy, so a thread waits for its own
// copies, issues fence.proxy.async and only then arrives on the stage's "full" mbarrier, two stages
// behind its newest copy.
//
// Roles in the CTA: NW worker threads (gather + epilogue), one TMA thread, one MMA thread.
// Every wait is bounded: when a spin budget runs out the thread records an error, raises the
// abort flag and keeps walking the loop nest without touching barriers' data, so the CTA still
// reaches its bar.sync points and exits.
#pragma once
#include "tiles_simt.cuh"

namespace tc {

constexpr int STAGES = 3;
constexpr int LAG = 2;                       // cp.async groups a worker keeps in flight
constexpr unsigned A_STAGE_BYTES = 128 * 128;
constexpr unsigned B_STAGE_BYTES = 256 * 128;
constexpr unsigned STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr unsigned NW = 256;                 // worker threads
constexpr unsigned TMA_THREAD = NW;          // lane 0 of warp 8
constexpr unsigned MMA_THREAD = NW + 32;     // lane 0 of warp 9
constexpr unsigned NTHREADS = NW + 64;
constexpr unsigned TMEM_COLS = 512;
// The epilogue's per-warp 4 KB transpose staging lives in the first 32 KB of the operand ring: all roles of the CTA move in
// lockstep, so when a block's accumulators are complete every stage has been read and no load of the next block is issued
// before the workers have finished (they fence the generic-proxy accesses against the next TMA writes before that barrier).
constexpr unsigned EPI_BYTES = 0;
constexpr unsigned RES_BYTES = (NW / 32) * 4096;   // per-warp landing slot for the other operand of a fused residual add

struct Shared {
    unsigned long long full[STAGES];
    unsigned long long empty[STAGES];
    unsigned long long landed[STAGES];   // TMA bytes of a stage have arrived
    unsigned long long accum;
    unsigned tmem_base;
    unsigned long long posted[2];     // scheduler -> executors: mailbox slot holds a tile
    unsigned long long finished[2];   // executors -> scheduler: every executor thread is done with the slot's tile
    unsigned mailbox[2];
    TileDev tile_desc[2];             // scheduler -> executors: the posted tile's descriptor (the scheduler has loaded it anyway)
    unsigned tile_nasm[2];            // ... and the index of its graph in the run
    unsigned long long res_full[NW / 32];   // per worker warp: its residual-operand box has landed
    // fused attention tile: queries / a key group / a value group have landed (TMA), the scores of a group are complete
    // (tcgen05.commit), the workers have written the group's probabilities to shared memory, the group's P x V MMAs are complete
    unsigned long long att_q, att_k, att_v, att_s, att_p, att_o;
    float partial[NW];        // K-attention row sums of the two column halves
};

struct PipeState {            // identical in every thread, carried across tiles
    unsigned it = 0;          // k-chunk iterations issued so far
    unsigned acc_phase = 0;   // accumulator barrier phase
    unsigned full_phase = 0;  // MMA thread: per-stage phase bits of the "full" barriers (not every layer uses them)
    unsigned res_uses = 0;    // worker warps: residual-operand boxes this warp has requested so far
    unsigned att_tiles = 0, att_groups = 0;   // fused attention tiles / key groups completed so far (barrier phases)
    bool dead = false;
};

// ---- PTX wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Non-blocking probe (try_wait may suspend the thread for a hardware-defined time; a polling loop
// that has other things to look at uses this one).
__device__ __forceinline__ bool mbar_test_wait(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and marks the run aborted) when the time budget runs out.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity, CtrlDev *ctrl, StatusHost *status, unsigned where) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    const unsigned long long budget = ctrl->pipe_ns;
    for (unsigned spin = 1;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 0u) {
            if (*(volatile unsigned *)&ctrl->abort) return false;
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (now - t0 > budget) break;
        }
    }
    if (atomicCAS(&ctrl->abort, 0u, (unsigned)ASPEN_B200_ERR_PIPE) == 0u) {
        status->info0 = where;
        status->info1 = blockIdx.x;
        status->status = ASPEN_B200_ERR_PIPE;
        __threadfence_system();
    }
    return false;
}

__device__ __forceinline__ void cp_async16(unsigned dst, const void *src, unsigned src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(unsigned dst, const void *src, unsigned src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(unsigned dst, const void *tmap, int x, int y, unsigned long long *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tma_load_3d(unsigned dst, const void *tmap, int x, int y, int z, unsigned long long *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(unsigned dst, const void *tmap, int x, int y, int z, int w, unsigned long long *bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(unsigned *holder, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float *v) {
    unsigned *r = reinterpret_cast<unsigned *>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart; version 1 (sm_100) in bits 46-47.
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3ffffu) >> 4);
    d |= (unsigned long long)1 << 16;                 // leading byte offset (unused for swizzled K-major)
    d |= (unsigned long long)(1024 >> 4) << 32;       // stride byte offset
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;                 // SWIZZLE_128B
    return d;
}
// D fp32, A/B tf32, both K-major, M = 128, N = n.
__device__ __forceinline__ unsigned umma_idesc(unsigned n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ unsigned swz(unsigned row, unsigned piece) { return row * 128u + ((piece ^ (row & 7u)) << 4); }

// Writes one 32 (tile columns n, one per lane) x 32 (rows m, in v[]) block of a warp's results.
// Each lane holds 32 consecutive m of ITS column, but global memory wants consecutive m from
// consecutive lanes, so the block is transposed through a 4 KB per-warp staging area (XOR-swizzled
// 16-byte pieces, conflict free both ways): every store instruction then covers four full 128-byte lines
// instead of 32 scattered 16-byte pieces.
__device__ __forceinline__ void store_block_coalesced(float *stage /*warp's 4 KB*/, const float *v, float *out_block /*(n = 0, m = 0)*/,
                                                      size_t ldc, unsigned n_valid, unsigned m_valid) {
    const unsigned lane = threadIdx.x & 31u;
    float4 *st = reinterpret_cast<float4 *>(stage);
    #pragma unroll
    for (unsigned j = 0; j < 8; j++) st[lane * 8u + (j ^ (lane & 7u))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    __syncwarp();
    const unsigned piece = lane & 7u, m = piece * 4u;
    #pragma unroll
    for (unsigned i = 0; i < 8; i++) {
        const unsigned n = i * 4u + (lane >> 3);
        const float4 val = st[n * 8u + (piece ^ (n & 7u))];
        if (n < n_valid) {
            float *dst = out_block + (size_t)n * ldc + m;
            if (m + 4u <= m_valid) *reinterpret_cast<float4 *>(dst) = val;
            else {
                if (m < m_valid) dst[0] = val.x;
                if (m + 1u < m_valid) dst[1] = val.y;
                if (m + 2u < m_valid) dst[2] = val.z;
            }
        }
    }
    __syncwarp();
}

// Same block store, plus the fused residual layer (ref src/tiled_kernels.c:503-541 computes it as a layer
// of its own): out2 = act(value + in2) for the same 32 x 32 block, read and written in the coalesced
// layout.  The eight loads of in2 are issued before the first store so they overlap.  `elide_own`: the
// pre-add value itself has no reader and is not stored.
__device__ __forceinline__ void store_block_residual(float *stage, const float *v, float *out_block, size_t ldc, unsigned n_valid,
                                                     unsigned m_valid, const float *in2_block, size_t ld_in2, float *out2_block,
                                                     size_t ld_out2, int act2, bool round2, bool elide_own) {
    const unsigned lane = threadIdx.x & 31u;
    float4 *st = reinterpret_cast<float4 *>(stage);
    #pragma unroll
    for (unsigned j = 0; j < 8; j++) st[lane * 8u + (j ^ (lane & 7u))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    __syncwarp();
    const unsigned piece = lane & 7u, m = piece * 4u;
    const bool full = m + 4u <= m_valid;
    float4 r[8];
    #pragma unroll
    for (unsigned i = 0; i < 8; i++) {
        const unsigned n = i * 4u + (lane >> 3);
        r[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n < n_valid) {
            const float *src = in2_block + (size_t)n * ld_in2 + m;
            if (full) r[i] = ldcg4(src);
            else {
                if (m < m_valid) r[i].x = ldcg1(src);
                if (m + 1u < m_valid) r[i].y = ldcg1(src + 1);
                if (m + 2u < m_valid) r[i].z = ldcg1(src + 2);
            }
        }
    }
    #pragma unroll
    for (unsigned i = 0; i < 8; i++) {
        const unsigned n = i * 4u + (lane >> 3);
        const float4 val = st[n * 8u + (piece ^ (n & 7u))];
        float4 o = make_float4(activate(val.x + r[i].x, act2), activate(val.y + r[i].y, act2), activate(val.z + r[i].z, act2),
                               activate(val.w + r[i].w, act2));
        if (round2) o = make_float4(tf32_round(o.x), tf32_round(o.y), tf32_round(o.z), tf32_round(o.w));
        if (n < n_valid) {
            float *dst = out_block + (size_t)n * ldc + m, *dst2 = out2_block + (size_t)n * ld_out2 + m;
            if (full) {
                if (!elide_own) *reinterpret_cast<float4 *>(dst) = val;
                *reinterpret_cast<float4 *>(dst2) = o;
            } else {
                if (m < m_valid) { if (!elide_own) dst[0] = val.x; dst2[0] = o.x; }
                if (m + 1u < m_valid) { if (!elide_own) dst[1] = val.y; dst2[1] = o.y; }
                if (m + 2u < m_valid) { if (!elide_own) dst[2] = val.z; dst2[2] = o.z; }
            }
        }
    }
    __syncwarp();
}

// Fused residual add, other operand by TMA.  The 32 (columns n) x 32 (rows m) block a warp needs for one epilogue chunk is a
// box of the other parent's matrix; lane 0 of the warp requests it into the warp's own 4 KB slot -- the first one before
// the block's main loop, so it lands while the MMAs run, each further one as soon as the previous has been read into
// registers -- and every lane then reads its own column's 32 values from shared memory (the 128-byte swizzle keeps the
// eight lanes of a quarter-warp on different banks).  The epilogue itself issues no global loads.
__device__ __forceinline__ void residual_request(unsigned slot_addr, const void *resmap, int m0, int n0, unsigned long long *bar) {
    mbar_arrive_expect_tx(bar, 4096u);
    tma_load_2d(slot_addr, resmap, m0, n0, bar);
}

// ---- per-layer operand description -------------------------------------------------------------
// How the two operands of a layer reach shared memory (chosen on the host, LayerDev::a_kind / b_kind):
//   X side  A_GATHER     worker threads, cp.async per 16-byte piece (4-byte pieces when IC % 4 != 0): strided
//                        convolutions, the 3-channel stem, connected layers over a padded parent
//           A_TMA        one 32 x 128 box per k-chunk straight from the parent's [columns][rows] matrix:
//                        matmul, 1x1 stride-1 convolution, attention, connected layers over an unpadded parent
//           A_TMA_FIXUP  stride-1 "same" convolution: tap (kh, kw) of 128 consecutive output pixels is the parent
//                        matrix shifted by (kh-p)*IW + (kw-p) columns, except where the tap leaves the image; the
//                        box is loaded shifted and the owner thread of each such row overwrites it with zeros
//           A_TMA_ROWS   convolution on the network input with <= 4 channels (the 7x7 stem): the input is kept as a
//                        zero-padded [sample][row][pixel][4] copy, the k axis is (kh, [kw][4] padded to 32), so
//                        one k-chunk of an output pixel is ONE contiguous 128-byte run of an input row, and 16 j
//                        consecutive output pixels of a row are a 3-D box (32 floats, 16 j pixels `stride` apart, 1
//                        row): two such boxes per chunk (cut at the end of an output row), no gather, no borders
//           A_TMA_IM2COL any convolution with IC % 32 == 0: the parent matrix seen as a 4-D tensor (channel, iw, ih,
//                        sample) with the convolution stride as TMA element stride.  One k-chunk = 32 channels of one
//                        tap; the 128 output pixels are cut into runs (rest of an output row, whole rows up to the end
//                        of the sample, ...) and each run is one box whose first pixel is (ow*s + kw - p, oh*s + kh - p):
//                        padding taps fall outside the tensor and arrive as zeros.  No gather, no fix-up; a handful
//                        of boxes per chunk, each run length with its own tensor map
//   W side  B_TMA        64-row boxes of the [rows][Kpad] weight copy
//           B_TMA_ACT    64-row boxes of the PARENT_1 activation matrix (attention keys)
//           B_GATHER     cp.async rows of PARENT_1 (attention keys whose head size is not a multiple of 32)
//           B_TRANSPOSED 4-byte cp.async transposing gather (attention values: W(m,k) = V[token k][feature m])
enum { A_GATHER = 0, A_TMA = 1, A_TMA_FIXUP = 2, A_TMA_ROWS = 3, A_TMA_IM2COL = 4 };
enum { B_GATHER = 0, B_TMA = 1, B_TMA_ACT = 2, B_TRANSPOSED = 3 };

struct Operands {
    const float *xrow;        // A_GATHER row-pointer layers: row n at xrow + n * xld
    size_t xld;
    bool conv;                // taps taken from L.in0 (convolution, connected)
    const float *wbase;       // gathered W: row m at wbase + m * wld (B_GATHER) or wbase[k * wld + m] (B_TRANSPOSED)
    size_t wld;
    unsigned w_rows;          // rows that exist (others read as zero)
    unsigned K, Kpad;
    int ax, ay;               // A_TMA: box coordinates of (column n0 = 0, k = 0)
    int bx, by;               // B_TMA / B_TMA_ACT: coordinates of (row 0 of the tile, k = 0)
    bool softmax;             // K-attention epilogue
    bool plain;               // V-attention epilogue: no bias / activation
    unsigned q0;              // K-attention: query index of tile column 0
};

__device__ __forceinline__ Operands make_operands(const LayerDev &L, const TileDev &T) {
    Operands o;
    o.conv = false; o.softmax = false; o.plain = false; o.q0 = 0;
    o.xrow = nullptr; o.xld = 0; o.wbase = nullptr; o.wld = 0; o.w_rows = T.tile_h;
    o.ax = 0; o.ay = (int)T.pos_w; o.bx = 0; o.by = (int)T.pos_h;
    switch (L.type) {
        case CONV_LAYER: case FC_LAYER:
            o.conv = true; o.K = L.K; o.Kpad = L.Kpad;
            break;
        case MATMUL_LAYER:
            o.xrow = L.in0 + (size_t)T.pos_w * L.ld0; o.xld = L.ld0; o.K = L.K; o.Kpad = L.Kpad;
            break;
        case K_ATTENTION_LAYER: {
            unsigned b = T.pos_w / (L.seq * L.heads), head = (T.pos_w % (L.seq * L.heads)) / L.seq;
            o.q0 = T.pos_w % L.seq;
            o.xrow = L.in0 + (size_t)(b * L.seq + o.q0) * L.ld0 + head * L.hd; o.xld = L.ld0;
            o.wbase = L.in1 + (size_t)(b * L.seq + T.pos_h) * L.ld1 + head * L.hd; o.wld = L.ld1;
            o.ax = (int)(head * L.hd); o.ay = (int)(b * L.seq + o.q0);
            o.bx = (int)(head * L.hd); o.by = (int)(b * L.seq + T.pos_h);
            o.K = L.hd; o.Kpad = (L.hd + 31u) & ~31u; o.softmax = true;
            break;
        }
        default: {   // V_ATTENTION_LAYER
            unsigned b = T.pos_w / L.seq, head = T.pos_h / L.hd, q0 = T.pos_w % L.seq;
            o.xrow = L.in0 + (size_t)((b * L.heads + head) * L.seq + q0) * L.ld0; o.xld = L.ld0;
            o.ay = (int)((b * L.heads + head) * L.seq + q0);
            o.wbase = L.in1 + (size_t)b * L.seq * L.ld1 + T.pos_h; o.wld = L.ld1;
            o.bx = (int)(b * L.seq); o.by = (int)T.pos_h;      // B_TMA_ACT: the transposed copy [feature][token]
            o.K = L.seq; o.Kpad = (L.seq + 31u) & ~31u; o.plain = true;
            break;
        }
    }
    return o;
}

// One ninst tile.  Called by all NTHREADS threads of the CTA.
static __device__ void tile_gemm(const LayerDev L, const TileDev T, const NasmDev &G, unsigned char *stage_mem, Shared *sh,
                          PipeState &ps, CtrlDev *ctrl, StatusHost *status) {
    const unsigned tid = threadIdx.x;
    const bool is_worker = tid < NW;
    const unsigned row = tid & 127u, half = (tid >> 7) & 1u;
    const Operands op = make_operands(L, T);
    const unsigned stage_base = smem_u32(stage_mem);
    const unsigned tmem = sh->tmem_base;
    const unsigned a_kind = L.a_kind, b_kind = L.b_kind;
    const bool a_tma = a_kind != A_GATHER, b_tma = b_kind == B_TMA || b_kind == B_TMA_ACT;
    const bool worker_work = (a_kind != A_TMA && a_kind != A_TMA_ROWS && a_kind != A_TMA_IM2COL) || !b_tma;      // workers write shared memory in this layer
    const void *amap = a_tma ? (const void *)((const unsigned char *)G.wmaps + (size_t)L.amap * 128) : nullptr;
    const void *bmap = b_tma ? (const void *)((const unsigned char *)G.wmaps + (size_t)L.wmap * 128) : nullptr;
    const bool vec_x = L.a_vec4 != 0;
    const bool res_tma = L.res_out != nullptr && L.resmap >= 0;
    const void *resmap = res_tma ? (const void *)((const unsigned char *)G.wmaps + (size_t)L.resmap * 128) : nullptr;

    // Activations were written with ordinary (generic proxy) stores, possibly by this very CTA a moment
    // ago; TMA reads them through the async proxy.
    if (tid == TMA_THREAD && a_tma) asm volatile("fence.proxy.async.global;" ::: "memory");
    if (res_tma && is_worker && (tid & 31u) == 0u) asm volatile("fence.proxy.async.global;" ::: "memory");

    const unsigned bw = L.bw;   // 128 except for convolutions whose blocks are whole output rows
    for (unsigned n0 = 0; n0 < T.tile_w; n0 += bw) {
        const unsigned rows_valid = min(bw, T.tile_w - n0);
        const bool row_ok = row < rows_valid;
        PixelWin pw = {0, 0, 0};
        const float *xr = nullptr;
        if (is_worker) {
            if (op.conv) pw = pixel_window(L, T.pos_w + n0 + row);
            else if (row_ok && a_kind == A_GATHER) xr = op.xrow + (size_t)(n0 + row) * op.xld;
        }
        for (unsigned ms = 0; ms < T.tile_h; ms += TMEM_COLS) {
            const unsigned cols_super = min(TMEM_COLS, T.tile_h - ms);
            unsigned arrived = ps.it;            // next iteration this worker still owes a "full" arrival for
            // fused residual add: ask for the first chunk's block of the other operand now, it lands under the main loop
            const unsigned wlane_base = ((tid >> 5) & 3u) * 32u;
            const bool res_live = res_tma && is_worker && rows_valid > wlane_base;          // this warp has columns in the block
            const unsigned res_slot = stage_base + STAGES * STAGE_BYTES + EPI_BYTES + (tid >> 5) * 4096u;
            const int res_m0 = (int)(T.pos_h + ms), res_n0 = (int)(T.pos_w + n0 + wlane_base);
            if (res_live && !ps.dead && half * 32u < cols_super && (tid & 31u) == 0u)
                residual_request(res_slot, resmap, res_m0 + (int)(half * 32u), res_n0, &sh->res_full[tid >> 5]);
            for (unsigned mp = 0; mp < cols_super; mp += 256) {
                const unsigned nb = min(256u, cols_super - mp);
                const unsigned NB = b_tma ? ((nb + 63u) & ~63u) : ((nb + 15u) & ~15u);
                for (unsigned kc = 0; kc < op.Kpad; kc += 32, ps.it++) {
                    const unsigned s = ps.it % STAGES, ph = (ps.it / STAGES) & 1u;
                    const unsigned sA = stage_base + s * STAGE_BYTES, sB = sA + A_STAGE_BYTES;
                    if (is_worker) {
                        if (!worker_work) continue;
                        if (a_kind == A_TMA_FIXUP) {
                            // the shifted box has landed: rows whose tap is outside the image become zero
                            if (!ps.dead && !mbar_wait(&sh->landed[s], ph, ctrl, status, 5)) ps.dead = true;
                            ps.dead = __any_sync(0xffffffffu, ps.dead);
                            if (!ps.dead && half == 0) {
                                const unsigned tap = kc / L.IC;
                                const int ih = pw.ih0 + (int)(tap / L.KW), iw = pw.iw0 + (int)(tap % L.KW);
                                if (ih < 0 || ih >= (int)L.IH || iw < 0 || iw >= (int)L.IW) {
                                    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                                    float4 *dst = reinterpret_cast<float4 *>(stage_mem + s * STAGE_BYTES + row * 128u);
                                    #pragma unroll
                                    for (int c = 0; c < 8; c++) dst[c] = z;
                                }
                            }
                            fence_proxy_async_smem();
                            if (!ps.dead) mbar_arrive(&sh->full[s]);
                            arrived = ps.it + 1;
                            continue;
                        }
                        if (!ps.dead && !mbar_wait(&sh->empty[s], ph ^ 1u, ctrl, status, 1)) ps.dead = true;
                        ps.dead = __any_sync(0xffffffffu, ps.dead);   // keep worker warps convergent on the failure path
                        if (!ps.dead) {
                            // ---- X side: this thread's half (4 pieces / 16 elements) of its row ----
                            if (a_kind == A_GATHER && row_ok) {
                                if (vec_x) {
                                    #pragma unroll
                                    for (unsigned c = 0; c < 4; c++) {
                                        const unsigned piece = half * 4 + c, k = kc + piece * 4;
                                        const float *src = L.in0;
                                        unsigned bytes = 0;
                                        if (k < op.K) {
                                            if (op.conv) {
                                                unsigned tap = k / L.IC, ic = k - tap * L.IC;
                                                const float *px = input_pixel(L, pw, (int)(tap / L.KW), (int)(tap % L.KW));
                                                if (px) { src = px + ic; bytes = 16; }
                                            } else { src = xr + k; bytes = 16; }
                                        }
                                        cp_async16(sA + swz(row, piece), src, bytes);
                                    }
                                } else {
                                    for (unsigned e = 0; e < 16; e++) {
                                        const unsigned kk = half * 16 + e, k = kc + kk;
                                        const float *src = L.in0;
                                        unsigned bytes = 0;
                                        if (k < op.K) {
                                            if (op.conv) {
                                                unsigned tap = k / L.IC, ic = k - tap * L.IC;
                                                const float *px = input_pixel(L, pw, (int)(tap / L.KW), (int)(tap % L.KW));
                                                if (px) { src = px + ic; bytes = 4; }
                                            } else { src = xr + k; bytes = 4; }
                                        }
                                        cp_async4(sA + swz(row, kk >> 2) + (kk & 3u) * 4u, src, bytes);
                                    }
                                }
                            }
                            // ---- W side when it is gathered ----
                            if (b_kind == B_GATHER) {
                                for (unsigned i = tid; i < NB * 8; i += NW) {
                                    const unsigned r = i >> 3, piece = i & 7u, k = kc + piece * 4, m = ms + mp + r;
                                    const bool ok = m < op.w_rows && k < op.K;
                                    cp_async16(sB + swz(r, piece), ok ? op.wbase + (size_t)m * op.wld + k : L.in1, ok ? 16u : 0u);
                                }
                            } else if (b_kind == B_TRANSPOSED) {
                                for (unsigned i = tid; i < NB * 32; i += NW) {
                                    const unsigned r = i % NB, kk = i / NB, k = kc + kk, m = ms + mp + r;
                                    const bool ok = m < op.w_rows && k < op.K;
                                    cp_async4(sB + swz(r, kk >> 2) + (kk & 3u) * 4u, ok ? op.wbase + (size_t)k * op.wld + m : L.in1, ok ? 4u : 0u);
                                }
                            }
                        }
                        cp_async_commit();
                        if (ps.it - arrived >= (unsigned)LAG) {       // copies of iteration `arrived` have landed
                            cp_async_wait<LAG>();
                            fence_proxy_async_smem();
                            if (!ps.dead) mbar_arrive(&sh->full[arrived % STAGES]);
                            arrived++;
                        }
                    } else if (tid == TMA_THREAD) {
                        if (!ps.dead && !mbar_wait(&sh->empty[s], ph ^ 1u, ctrl, status, 2)) ps.dead = true;
                        if (!ps.dead) {
                            const unsigned bytes = (a_tma ? (a_kind == A_TMA_IM2COL ? (bw != 128u ? bw : rows_valid) * 128u : A_STAGE_BYTES) : 0u) + (b_tma ? NB * 128u : 0u);
                            if (bytes) mbar_arrive_expect_tx(&sh->landed[s], bytes);
                            else mbar_arrive(&sh->landed[s]);
                            if (a_kind == A_TMA_ROWS) {
                                // chunk kc / 32 is filter row kh.  The 128 pixels are cut where an output row ends; a run of
                                // 16 j pixels uses the j-th of the layer's consecutive tensor maps (box of 16 j pixels).
                                const unsigned hw = L.OH * L.OW;
                                #pragma unroll 1
                                for (unsigned done = 0; done < 128u;) {
                                    const unsigned n = T.pos_w + n0 + done;
                                    const unsigned b = n / hw, r = n - b * hw, oh = r / L.OW, ow = r - oh * L.OW;
                                    const unsigned len = min(128u - done, L.OW - ow);
                                    tma_load_3d(sA + done * 128u, (const unsigned char *)amap + (size_t)(len / 16u - 1u) * 128, 0, (int)ow,
                                                (int)(b * L.PH + oh * L.stride + (kc >> 5)), &sh->landed[s]);
                                    done += len;
                                }
                            } else if (a_kind == A_TMA_IM2COL) {
                                const unsigned tap = kc / L.IC, c0 = kc - tap * L.IC, kh = tap / L.KW, kw = tap - kh * L.KW;
                                const unsigned hw = L.OH * L.OW;
                                if (bw != 128u) {
                                    // the block is whole output rows of one sample, or whole samples: one box
                                    const unsigned n = T.pos_w + n0;
                                    const unsigned b = n / hw, r = n - b * hw, oh = r / L.OW;
                                    tma_load_4d(sA, (const unsigned char *)amap + (size_t)L.one_box * 128, (int)c0, (int)kw - (int)L.pad,
                                                (int)(oh * L.stride + kh) - (int)L.pad, (int)b, &sh->landed[s]);
                                } else
                                #pragma unroll 1
                                for (unsigned done = 0; done < rows_valid;) {
                                    const unsigned n = T.pos_w + n0 + done, rem = rows_valid - done;
                                    const unsigned b = n / hw, r = n - b * hw, oh = r / L.OW, ow = r - oh * L.OW;
                                    unsigned len, mi;
                                    if (ow != 0u || rem < L.OW) { len = min(rem, L.OW - ow); mi = len - 1u; }          // (rest of) one output row
                                    else { const unsigned k = min(rem / L.OW, L.OH - oh); len = k * L.OW; mi = L.OW + k - 2u; }   // k whole rows
                                    tma_load_4d(sA + done * 128u, (const unsigned char *)amap + (size_t)mi * 128, (int)c0,
                                                (int)(ow * L.stride + kw) - (int)L.pad, (int)(oh * L.stride + kh) - (int)L.pad, (int)b, &sh->landed[s]);
                                    done += len;
                                }
                            } else if (a_tma) {
                                int x = op.ax + (int)kc, y = op.ay + (int)n0;
                                if (a_kind == A_TMA_FIXUP) {
                                    const unsigned tap = kc / L.IC;
                                    x = (int)(kc - tap * L.IC);
                                    y += ((int)(tap / L.KW) - (int)L.pad) * (int)L.IW + ((int)(tap % L.KW) - (int)L.pad);
                                }
                                tma_load_2d(sA, amap, x, y, &sh->landed[s]);
                            }
                            if (b_tma)
                                for (unsigned j = 0; j < NB; j += 64)
                                    tma_load_2d(sB + j * 128u, bmap, op.bx + (int)kc, op.by + (int)(ms + mp + j), &sh->landed[s]);
                        }
                    } else if (tid == MMA_THREAD) {
                        if (!ps.dead && !mbar_wait(&sh->landed[s], ph, ctrl, status, 3)) ps.dead = true;
                        if (worker_work) {
                            if (!ps.dead && !mbar_wait(&sh->full[s], (ps.full_phase >> s) & 1u, ctrl, status, 6)) ps.dead = true;
                            ps.full_phase ^= 1u << s;
                        }
                        if (!ps.dead) {
                            tc_fence_after();
                            const unsigned long long adesc = umma_desc(sA), bdesc = umma_desc(sB);
                            const unsigned idesc = umma_idesc(NB);
                            #pragma unroll
                            for (unsigned k8 = 0; k8 < 4; k8++)
                                tc_mma_tf32(tmem + mp, adesc + 2ull * k8, bdesc + 2ull * k8, idesc, (kc | k8) != 0u);
                            tc_commit(&sh->empty[s]);
                        }
                    }
                }
            }
            // ---- all k-chunks of this 128 x cols_super block are issued ----
            if (tid == MMA_THREAD && !ps.dead) tc_commit(&sh->accum);
            if (is_worker) {
                if (worker_work && a_kind != A_TMA_FIXUP) {
                    cp_async_wait<0>();
                    fence_proxy_async_smem();
                    for (; arrived != ps.it; arrived++)
                        if (!ps.dead) mbar_arrive(&sh->full[arrived % STAGES]);
                }
                if (!ps.dead && !mbar_wait(&sh->accum, ps.acc_phase, ctrl, status, 4)) ps.dead = true;
                ps.dead = __any_sync(0xffffffffu, ps.dead);
                tc_fence_after();
                // ---- epilogue: thread = output column n0 + row, this half's 32-wide row chunks ----
                const unsigned lane_base = ((tid >> 5) & 3u) * 32u;
                const unsigned nchunk = (cols_super + 31u) >> 5;
                // block (n = first column of this warp's 32, m = ms) of the output matrix
                float *oblk = L.out + (size_t)(T.pos_w + n0 + lane_base) * L.ldc + T.pos_h + ms;
                const unsigned n_valid = rows_valid > lane_base ? rows_valid - lane_base : 0u;
                float *epi = reinterpret_cast<float *>(stage_mem) + (tid >> 5) * 1024u;
                float v[32];
                if (op.softmax) {
                    // scores -> mask -> / sqrt(hd) -> exp, normalised by the column sum (ref src/tiled_kernels.c:859-876)
                    // fast exponential and reciprocals: this path is the TF32 one, whose bound is 1e-2 of the layer's maximum
                    const float inv_scale = 1.f / sqrtf((float)L.hd);
                    const unsigned q = op.q0 + n0 + row;
                    float sum = 0.f;
                    for (unsigned c = half; c < nchunk; c += 2) {
                        if (!ps.dead) tmem_ld32(tmem + (lane_base << 16) + c * 32u, v);
                        #pragma unroll
                        for (unsigned j = 0; j < 32; j++) {
                            const unsigned m = ms + c * 32u + j;
                            if (m < T.tile_h) {
                                float x = (L.masked && (T.pos_h + m) > q) ? -1e10f : v[j];
                                sum += __expf(x * inv_scale);
                            }
                        }
                    }
                    sh->partial[tid] = sum;
                    worker_barrier(NW);
                    sum = sh->partial[row] + sh->partial[row + 128u];
                    const float inv_sum = 1.f / sum;
                    for (unsigned c = half; c < nchunk; c += 2) {
                        if (!ps.dead) tmem_ld32(tmem + (lane_base << 16) + c * 32u, v);
                        #pragma unroll
                        for (unsigned j = 0; j < 32; j++) {
                            const unsigned m = ms + c * 32u + j;
                            float x = (L.masked && (T.pos_h + m) > q) ? -1e10f : v[j];
                            v[j] = store_round(__expf(x * inv_scale) * inv_sum, L);
                        }
                        if (!ps.dead) store_block_coalesced(epi, v, oblk + c * 32u, L.ldc, n_valid, min(32u, cols_super - c * 32u));
                    }
                    worker_barrier(NW);   // partial[] is reused by the next block
                } else {
                    const float *bias = (!op.plain && L.bias) ? L.bias + T.pos_h + ms : nullptr;
                    const bool bias_vec = bias && ((reinterpret_cast<uintptr_t>(bias) & 15u) == 0u);
                    const int act = L.act;
                    const bool rnd = L.round_out != 0;
                    for (unsigned c = half; c < nchunk; c += 2) {
                        if (!ps.dead) tmem_ld32(tmem + (lane_base << 16) + c * 32u, v);
                        const unsigned valid = min(32u, cols_super - c * 32u);
                        if (bias) {
                            if (bias_vec && valid == 32u) {
                                #pragma unroll
                                for (unsigned j = 0; j < 32; j += 4) {
                                    const float4 b4 = __ldg(reinterpret_cast<const float4 *>(bias + c * 32u + j));
                                    v[j] += b4.x; v[j + 1] += b4.y; v[j + 2] += b4.z; v[j + 3] += b4.w;
                                }
                            } else {
                                #pragma unroll
                                for (unsigned j = 0; j < 32; j++)
                                    if (j < valid) v[j] += __ldg(bias + c * 32u + j);
                            }
                        }
                        if (!op.plain) {
                            if (act == RELU) {
                                #pragma unroll
                                for (unsigned j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
                            } else if (act == GELU) {
                                #pragma unroll
                                for (unsigned j = 0; j < 32; j++) v[j] = gelu_erf_fast(v[j]);
                            } else if (act == GELU_ACCURATE) {
                                #pragma unroll
                                for (unsigned j = 0; j < 32; j++) v[j] = gelu_tanh_fast(v[j]);
                            } else if (act != NO_ACTIVATION && act != LINEAR) {
                                #pragma unroll
                                for (unsigned j = 0; j < 32; j++) v[j] = activate(v[j], act);
                            }
                        }
                        if (rnd) {
                            #pragma unroll
                            for (unsigned j = 0; j < 32; j++) v[j] = tf32_round(v[j]);
                        }
                        if (L.vt_out && !ps.dead && row < rows_valid) {
                            // transposed copy for an attention_v consumer: lanes hold consecutive columns, so each of the 32
                            // stores of a warp covers one full 128-byte line of a feature's row
                            float *vt = L.vt_out + (size_t)(T.pos_h + ms + c * 32u) * L.vt_ld + T.pos_w + n0 + row;
                            #pragma unroll
                            for (unsigned j = 0; j < 32; j++)
                                if (j < valid) vt[(size_t)j * L.vt_ld] = v[j];
                        }
                        if (res_live) {
                            // the other operand's block is in this warp's slot: own column = row `lane` of the box
                            if (!ps.dead && !mbar_wait(&sh->res_full[tid >> 5], ps.res_uses & 1u, ctrl, status, 11)) ps.dead = true;
                            ps.dead = __any_sync(0xffffffffu, ps.dead);
                            ps.res_uses++;
                            float4 r[8];
                            const unsigned lane = tid & 31u;
                            const float4 *slot = reinterpret_cast<const float4 *>(stage_mem + STAGES * STAGE_BYTES + EPI_BYTES + (tid >> 5) * 4096u + lane * 128u);
                            #pragma unroll
                            for (unsigned q = 0; q < 8; q++) r[q] = slot[q ^ (lane & 7u)];
                            __syncwarp();
                            if (!ps.dead && c + 2u < nchunk && lane == 0u)
                                residual_request(res_slot, resmap, res_m0 + (int)((c + 2u) * 32u), res_n0, &sh->res_full[tid >> 5]);
                            if (!ps.dead) {
                                if (!L.res_elide) store_block_coalesced(epi, v, oblk + c * 32u, L.ldc, n_valid, valid);
                                const int act2 = L.res_act;
                                #pragma unroll
                                for (unsigned q = 0; q < 8; q++) { v[4 * q] += r[q].x; v[4 * q + 1] += r[q].y; v[4 * q + 2] += r[q].z; v[4 * q + 3] += r[q].w; }
                                if (act2 == RELU) {
                                    #pragma unroll
                                    for (unsigned j = 0; j < 32; j++) v[j] = v[j] > 0.f ? v[j] : 0.f;
                                } else if (act2 != NO_ACTIVATION && act2 != LINEAR) {
                                    #pragma unroll
                                    for (unsigned j = 0; j < 32; j++) v[j] = activate(v[j], act2);
                                }
                                if (L.res_round) {
                                    #pragma unroll
                                    for (unsigned j = 0; j < 32; j++) v[j] = tf32_round(v[j]);
                                }
                                const size_t colg = T.pos_w + n0 + lane_base, mg = T.pos_h + ms + c * 32u;
                                store_block_coalesced(epi, v, L.res_out + colg * L.res_ld_out + mg, L.res_ld_out, n_valid, valid);
                            }
                        } else if (!ps.dead) {
                            if (L.res_out) {
                                const size_t col0 = T.pos_w + n0 + lane_base, m0 = T.pos_h + ms + c * 32u;
                                store_block_residual(epi, v, oblk + c * 32u, L.ldc, n_valid, valid, L.res_in + col0 * L.res_ld_in + m0, L.res_ld_in,
                                                     L.res_out + col0 * L.res_ld_out + m0, L.res_ld_out, L.res_act, L.res_round != 0, L.res_elide != 0);
                            } else store_block_coalesced(epi, v, oblk + c * 32u, L.ldc, n_valid, valid);
                        }
                    }
                }
                fence_proxy_async_smem();     // staging reads and writes of the ring's memory, before the next block's TMA writes
                tc_fence_before();
            }
            ps.acc_phase ^= 1u;
            // The MMA thread must not overwrite the accumulators before every epilogue thread has read them.
            __syncwarp();
            asm volatile("bar.sync 2, %0;" ::"r"(NTHREADS) : "memory");
            if (tid == MMA_THREAD) tc_fence_after();
        }
    }
}

// ---- attention_k + attention_v as ONE tile -------------------------------------------------------------
// An attention_v tile -- one head's features for up to 128 queries of one sample -- computes its own probabilities
// instead of reading them back (ref src/tiled_kernels.c:784-932 and 934-1038 are two layers with the seq x seq matrix
// between them).  Per group of 128 keys:
//     S = Q K^T           tcgen05.mma, M = 128 queries, N = 128 keys, K = head size; Q and K by TMA from the projections
//     e = exp(mask(S) / sqrt(hd))   by the thread that owns the query row, straight from TMEM; row sums stay in registers
//     P (TF32, unnormalised) -> shared memory in the K-major swizzled operand layout
//     O += P V            tcgen05.mma, M = 128, N = head size, K = 128 keys; V by TMA from the transposed copy
// and at the end O / rowsum is stored.  The reference's softmax subtracts no maximum, so groups need no rescaling.
// With a causal mask the groups that lie entirely above the tile's queries are skipped.  When every hidden state must
// stay readable (the host allows that with one key group only) the normalised probabilities are also written to the
// attention_k layer's matrix, recomputed from the scores that are still in TMEM.
// The operand ring (and the residual slots behind it) is carved up for this tile: Q 32 KB | K 32 KB | P 64 KB | V 32 KB;
// the epilogue's transpose staging reuses the Q buffer, which nothing reads once the last MMA has completed.
// Every barrier completes once per key group (att_q once per tile), in order, so the parity of a completion follows from
// counts every thread keeps: no role has to track which barriers it waited on.
constexpr unsigned ATT_Q = 0u, ATT_K = 32768u, ATT_P = 65536u, ATT_V = 131072u, ATT_EPI = 0u;
static_assert(ATT_V + 32768u <= STAGES * STAGE_BYTES + RES_BYTES, "the attention tile's buffers must fit the ring plus the residual slots");
constexpr unsigned ATT_ACC_O = 256u;      // TMEM column of the output accumulator (scores use columns 0..127)

// The function is deliberately NOT inlined into the persistent kernel and takes everything by value: inlined, its register
// needs pushed the contraction tile's main loop into spills (the whole kernel ran 45 % slower, attention layer or not); a
// call that takes references to the kernel's own state forces that state into local memory (worse still).  It returns the
// `dead` flag; the caller advances the two phase counters.
struct AttnArgs {     // what the tile needs of its layer descriptor
    unsigned seq, hd, heads, masked, ldc, round_out, att_p_ld, att_p_round;
    float *out, *att_p_out;
    const void *qmap, *kmap, *vmap;
};
struct AttnPipe { unsigned att_tiles, att_groups; bool dead; };

static __device__ __noinline__ bool tile_attention(const AttnArgs L, const TileDev T, unsigned char *stage_mem, Shared *sh,
                                                   AttnPipe ps, CtrlDev *ctrl, StatusHost *status) {
    const unsigned tid = threadIdx.x;
    const bool is_worker = tid < NW;
    const unsigned row = tid & 127u, half = (tid >> 7) & 1u;
    const unsigned base = smem_u32(stage_mem), tmem = sh->tmem_base;
    const unsigned seq = L.seq, hd = L.hd, qchunks = hd >> 5;
    const unsigned b = T.pos_w / seq, q0 = T.pos_w - b * seq, head = T.pos_h / hd;
    const unsigned nq = T.tile_w;
    const void *qmap = L.qmap, *kmap = L.kmap, *vmap = L.vmap;
    // key groups of 128; with a causal mask nothing beyond the last query's own position contributes
    const unsigned last_key = L.masked ? min(seq, q0 + nq) : seq;
    const unsigned groups = (last_key + 127u) >> 7;
    const float inv_scale = 1.f / sqrtf((float)hd);
    const unsigned lane_base = ((tid >> 5) & 3u) * 32u;
    const unsigned q = q0 + row;
    float rowsum = 0.f;
    // parity of the completion that belongs to key group g of THIS tile
    #define ATT_PAR(g) ((ps.att_groups + (g)) & 1u)

    if (tid == TMA_THREAD) asm volatile("fence.proxy.async.global;" ::: "memory");
    for (unsigned g = 0; g < groups; g++) {
        const unsigned key0 = g << 7;
        if (tid == TMA_THREAD) {
            if (g == 0 && !ps.dead) {
                mbar_arrive_expect_tx(&sh->att_q, qchunks * A_STAGE_BYTES);
                for (unsigned c = 0; c < qchunks; c++)
                    tma_load_2d(base + ATT_Q + c * A_STAGE_BYTES, qmap, (int)(head * hd + c * 32u), (int)(b * seq + q0), &sh->att_q);
            }
            // the key buffer is free once the previous group's scores are complete, the value buffer once its P x V is
            if (g > 0 && !ps.dead && !mbar_wait(&sh->att_s, ATT_PAR(g - 1u), ctrl, status, 12)) ps.dead = true;
            if (!ps.dead) {
                mbar_arrive_expect_tx(&sh->att_k, qchunks * A_STAGE_BYTES);
                for (unsigned c = 0; c < qchunks; c++)
                    for (unsigned j = 0; j < 128u; j += 64u)
                        tma_load_2d(base + ATT_K + c * A_STAGE_BYTES + j * 128u, kmap, (int)(head * hd + c * 32u), (int)(b * seq + key0 + j), &sh->att_k);
            }
            if (g > 0 && !ps.dead && !mbar_wait(&sh->att_o, ATT_PAR(g - 1u), ctrl, status, 13)) ps.dead = true;
            if (!ps.dead) {
                mbar_arrive_expect_tx(&sh->att_v, 4u * 8192u);
                for (unsigned c = 0; c < 4u; c++)
                    tma_load_2d(base + ATT_V + c * 8192u, vmap, (int)(b * seq + key0 + c * 32u), (int)T.pos_h, &sh->att_v);
            }
        } else if (tid == MMA_THREAD) {
            if (g == 0 && !ps.dead && !mbar_wait(&sh->att_q, ps.att_tiles & 1u, ctrl, status, 14)) ps.dead = true;
            if (!ps.dead && !mbar_wait(&sh->att_k, ATT_PAR(g), ctrl, status, 15)) ps.dead = true;
            if (!ps.dead) {
                tc_fence_after();
                const unsigned idesc = umma_idesc(128u);
                for (unsigned c = 0; c < qchunks; c++) {
                    const unsigned long long adesc = umma_desc(base + ATT_Q + c * A_STAGE_BYTES), bdesc = umma_desc(base + ATT_K + c * A_STAGE_BYTES);
                    #pragma unroll
                    for (unsigned k8 = 0; k8 < 4; k8++) tc_mma_tf32(tmem, adesc + 2ull * k8, bdesc + 2ull * k8, idesc, (c | k8) != 0u);
                }
                tc_commit(&sh->att_s);
            }
            // probabilities of the group in shared memory (the workers have also finished reading the scores), values landed
            if (!ps.dead && !mbar_wait(&sh->att_p, ATT_PAR(g), ctrl, status, 16)) ps.dead = true;
            if (!ps.dead && !mbar_wait(&sh->att_v, ATT_PAR(g), ctrl, status, 17)) ps.dead = true;
            if (!ps.dead) {
                tc_fence_after();
                const unsigned idesc = umma_idesc(hd);
                for (unsigned c = 0; c < 4u; c++) {
                    const unsigned long long adesc = umma_desc(base + ATT_P + c * A_STAGE_BYTES), bdesc = umma_desc(base + ATT_V + c * 8192u);
                    #pragma unroll
                    for (unsigned k8 = 0; k8 < 4; k8++) tc_mma_tf32(tmem + ATT_ACC_O, adesc + 2ull * k8, bdesc + 2ull * k8, idesc, (g | c | k8) != 0u);
                }
                tc_commit(&sh->att_o);
            }
        } else if (is_worker) {
            if (!ps.dead && !mbar_wait(&sh->att_s, ATT_PAR(g), ctrl, status, 18)) ps.dead = true;
            // the previous group's P x V must have read the probability buffer before it is overwritten
            if (g > 0 && !ps.dead && !mbar_wait(&sh->att_o, ATT_PAR(g - 1u), ctrl, status, 19)) ps.dead = true;
            ps.dead = __any_sync(0xffffffffu, ps.dead);
            tc_fence_after();
            #pragma unroll 1
            for (unsigned i = 0; i < 2; i++) {
                const unsigned c = half + 2u * i;                                   // chunk of 32 keys inside the group
                float v[32];
                if (!ps.dead) tmem_ld32(tmem + (lane_base << 16) + c * 32u, v);
                #pragma unroll
                for (unsigned j = 0; j < 32; j++) {
                    const unsigned key = key0 + c * 32u + j;
                    float x = 0.f;
                    if (key < seq) x = __expf(((L.masked && key > q) ? -1e10f : v[j]) * inv_scale);
                    rowsum += x;
                    v[j] = tf32_round(x);
                }
                float4 *dst = reinterpret_cast<float4 *>(stage_mem + ATT_P + c * A_STAGE_BYTES + row * 128u);
                #pragma unroll
                for (unsigned p = 0; p < 8; p++) dst[p ^ (row & 7u)] = make_float4(v[4 * p], v[4 * p + 1], v[4 * p + 2], v[4 * p + 3]);
            }
            fence_proxy_async_smem();
            tc_fence_before();
            if (!ps.dead) mbar_arrive(&sh->att_p);
        }
    }
    if (is_worker) {
        // row sum over both halves of the row, then the output block
        sh->partial[tid] = rowsum;
        worker_barrier(NW);
        const float inv_sum = 1.f / (sh->partial[row] + sh->partial[row + 128u]);
        if (!ps.dead && !mbar_wait(&sh->att_o, ATT_PAR(groups - 1u), ctrl, status, 20)) ps.dead = true;
        ps.dead = __any_sync(0xffffffffu, ps.dead);
        tc_fence_after();
        const unsigned n_valid = nq > lane_base ? nq - lane_base : 0u;
        float *epi = reinterpret_cast<float *>(stage_mem + ATT_EPI) + (tid >> 5) * 1024u;
        float v[32];
        if (half * 32u < hd) {
            if (!ps.dead) tmem_ld32(tmem + (lane_base << 16) + ATT_ACC_O + half * 32u, v);
            #pragma unroll
            for (unsigned j = 0; j < 32; j++) v[j] = L.round_out ? tf32_round(v[j] * inv_sum) : v[j] * inv_sum;
            float *oblk = L.out + (size_t)(T.pos_w + lane_base) * L.ldc + T.pos_h + half * 32u;
            if (!ps.dead) store_block_coalesced(epi, v, oblk, L.ldc, n_valid, min(32u, T.tile_h - half * 32u));
        }
        if (L.att_p_out) {
            // the attention_k layer's own matrix: column (b, head, query), rows = keys; one group, its scores are still in TMEM
            #pragma unroll 1
            for (unsigned c = half; c * 32u < seq; c += 2u) {
                if (!ps.dead) tmem_ld32(tmem + (lane_base << 16) + c * 32u, v);
                #pragma unroll
                for (unsigned j = 0; j < 32; j++) {
                    const unsigned key = c * 32u + j;
                    float x = 0.f;
                    if (key < seq) x = __expf(((L.masked && key > q) ? -1e10f : v[j]) * inv_scale) * inv_sum;
                    v[j] = L.att_p_round ? tf32_round(x) : x;
                }
                float *pblk = L.att_p_out + (size_t)((b * L.heads + head) * seq + q0 + lane_base) * L.att_p_ld + c * 32u;
                if (!ps.dead) store_block_coalesced(epi, v, pblk, L.att_p_ld, n_valid, min(32u, seq - c * 32u));
            }
        }
        worker_barrier(NW);           // partial[] is reused by the next tile
        fence_proxy_async_smem();     // generic accesses to the ring's memory, before the next tile's TMA writes
        tc_fence_before();
    }
    #undef ATT_PAR
    __syncwarp();
    asm volatile("bar.sync 2, %0;" ::"r"(NTHREADS) : "memory");
    if (tid == MMA_THREAD) tc_fence_after();
    return ps.dead;
}

// Key groups the fused attention tile walks for tile T (the caller advances its phase counter by this).
__device__ __forceinline__ unsigned attention_groups(unsigned seq, unsigned masked, const TileDev &T) {
    const unsigned q0 = T.pos_w % seq;
    const unsigned last_key = masked ? min(seq, q0 + T.tile_w) : seq;
    return (last_key + 127u) >> 7;
}

}  // namespace tc
