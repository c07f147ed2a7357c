// Persistent device-side dataflow scheduler: the B200 counterpart of the reference's DSE worker
// loop (dse_schedule, ref src/dse.c:20-108) and ready pool (ref src/rpool.c:390-685).
//
// One CTA per SM stays resident for a whole run.  Its control warp
//   pops a ready tile      (rpool_fetch_ninsts)     ticket = atomicAdd(head); wait for queue[ticket]
//   lets the CTA run it    (switch on layer type, ref src/dse.c:39-79)
//   accounts completion    (layer counter -> layers-completed counter -> completed flag, ref src/dse.c:80-106)
//   updates the children   (update_children_but_prioritize_dse_target, ref src/dse.c:363-401):
//                          atomicAdd on each child's dependency counter; a child whose last parent
//                          this was becomes ready; the first such child is kept as this CTA's next
//                          tile (depth first, no queue round trip), the others are pushed.
// There is no kernel boundary and no barrier between layers: a tile fires as soon as its own
// parent tiles are complete.
//
// The queue is a ticket ring: every tile is pushed at most once per run, so a ring of `total`
// slots never wraps; slot value = global tile id + 1, 0 = not yet filled.  A popper that holds a
// ticket whose slot is still empty waits -- bounded: when no tile anywhere completes for
// `stall_ns` it records ASPEN_B200_ERR_STALL, raises the abort flag and every CTA leaves.
//
// Memory ordering: tile data is written by the worker threads; bar.sync orders it before the
// control warp's fence.acq_rel.gpu + relaxed atomicAdd on the child counter (release).  The CTA
// whose increment completes the count fences again after the atomic (acquiring every earlier
// parent's data through the counter's RMW chain) before it publishes or keeps the child.
#pragma once
#include "tiles_tc.cuh"

namespace sched {

constexpr unsigned PROF_LAYERS = 256;
constexpr unsigned PROF_SLOTS = 2 + 2 * PROF_LAYERS;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by lane 0 of the control warp.  Returns a global tile id or ASPEN_TILE_NONE.
__device__ unsigned pop_ready(CtrlDev *ctrl, const unsigned *queue, StatusHost *status) {
    if (ld_relaxed(&ctrl->stop) || ld_relaxed(&ctrl->abort)) return ASPEN_TILE_NONE;
    const unsigned ticket = atomicAdd(&ctrl->head, 1u);
    const unsigned total = ctrl->total, cap = ctrl->cap;
    if (ticket >= cap) return ASPEN_TILE_NONE;          // every tile that can ever be pushed already has an owner
    unsigned last_done = ld_relaxed(&ctrl->done);
    unsigned long long t_last = global_ns();
    const unsigned long long window = ctrl->stall_ns;
    for (unsigned spin = 0;; spin++) {
        unsigned v = ld_acquire(&queue[ticket]);
        if (v != 0u) return v - 1u;
        unsigned done = ld_relaxed(&ctrl->done);
        if (done >= total) return ASPEN_TILE_NONE;      // run finished; this ticket is never filled
        if (ld_relaxed(&ctrl->abort) || ld_relaxed(&ctrl->stop)) return ASPEN_TILE_NONE;
        if ((spin & 63u) == 63u) {
            unsigned long long now = global_ns();
            if (done != last_done) { last_done = done; t_last = now; }
            else if (now - t_last > window) {
                if (atomicCAS(&ctrl->abort, 0u, (unsigned)ASPEN_B200_ERR_STALL) == 0u) {
                    status->info0 = ticket;
                    status->info1 = done;
                    status->status = ASPEN_B200_ERR_STALL;
                    __threadfence_system();
                }
                return ASPEN_TILE_NONE;
            }
        }
        __nanosleep(spin < 16u ? 32u : 256u);
    }
}

// Called by the whole (converged) control warp after the tile's data is complete.
// Returns the global id of a child this CTA should run next, or ASPEN_TILE_NONE.
__device__ unsigned complete_tile(const NasmDev &G, unsigned local, CtrlDev *ctrl, unsigned *queue, StatusHost *status) {
    const unsigned lane = threadIdx.x & 31u;
    const TileDev T = G.tiles[local];
    __threadfence();                                     // release: this tile's output
    if (lane == 0) {
        unsigned d = atomicAdd(&G.layer_done[T.layer], 1u);
        if (d + 1u == G.layer_tiles[T.layer]) {
            unsigned l = atomicAdd(G.layers_completed, 1u);
            if (l + 1u == G.n_layers) {
                __threadfence_system();
                *G.completed = 1u;                       // mapped host flag: the nasm is complete
            }
        }
    }
    unsigned next = ASPEN_TILE_NONE;
    for (unsigned base = 0; base < T.child_cnt; base += 32u) {
        const unsigned idx = base + lane;
        unsigned child = ASPEN_TILE_NONE;
        bool ready = false;
        if (idx < T.child_cnt) {
            child = G.children[T.child_off + idx];
            unsigned old = atomicAdd(&G.dep[child], 1u);
            ready = old + 1u == G.tiles[child].need;
        }
        unsigned mask = __ballot_sync(0xffffffffu, ready);
        if (mask == 0u) continue;
        __threadfence();                                 // acquire the other parents' outputs (through the counters), then publish
        if (next == ASPEN_TILE_NONE) {
            const unsigned first = __ffs(mask) - 1u;
            next = __shfl_sync(0xffffffffu, child, first) + G.tile_base;
            mask &= ~(1u << first);
            if (lane == first) ready = false;
        }
        const unsigned n_push = __popc(mask);
        if (n_push) {
            unsigned pos = 0;
            if (lane == 0) pos = atomicAdd(&ctrl->tail, n_push);
            pos = __shfl_sync(0xffffffffu, pos, 0);
            if (ready) {
                const unsigned rank = __popc(mask & ((1u << lane) - 1u));
                if (pos + rank < ctrl->cap)
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&queue[pos + rank]), "r"(child + G.tile_base + 1u) : "memory");
            }
        }
    }
    if (lane == 0) {
        unsigned d = atomicAdd(&ctrl->done, 1u);
        if (((d + 1u) & 1023u) == 0u || d + 1u == ctrl->total) status->tiles_done = d + 1u;
    }
    return __shfl_sync(0xffffffffu, next, 0);
}

// Resets the counters of every graph in the run and seeds the queue with the tiles that only
// depend on input tiles (push_first_layer_to_rpool, ref src/dse.c:443-470).
__global__ void arm_kernel(NasmDev *nasms, CtrlDev *ctrl, unsigned *queue, unsigned total, unsigned n_init_total,
                           unsigned n_input_total, unsigned long long stall_ns, unsigned long long pipe_ns) {
    const unsigned stride = gridDim.x * blockDim.x, t0 = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned n_nasm = ctrl->n_nasm;
    for (unsigned i = t0; i < total; i += stride) queue[i] = 0u;
    __threadfence();
    for (unsigned g = 0; g < n_nasm; g++) {
        const NasmDev G = nasms[g];
        for (unsigned i = t0; i < G.n_tiles; i += stride) G.dep[i] = G.dep_init[i];
        for (unsigned i = t0; i < G.n_layers; i += stride) G.layer_done[i] = i == 0 ? G.layer_tiles[0] : 0u;
        if (t0 == 0) { *G.layers_completed = 1u; *G.completed = 0u; }
    }
    if (t0 == 0) {
        ctrl->head = 0u; ctrl->tail = n_init_total; ctrl->done = n_input_total; ctrl->total = total; ctrl->cap = total;
        ctrl->abort = 0u; ctrl->stop = 0u; ctrl->stall_ns = stall_ns; ctrl->pipe_ns = pipe_ns;
    }
}
// Second step of arming (after every slot was cleared): write the initial ready tiles.
__global__ void seed_kernel(NasmDev *nasms, CtrlDev *ctrl, unsigned *queue) {
    const unsigned stride = gridDim.x * blockDim.x, t0 = blockIdx.x * blockDim.x + threadIdx.x;
    for (unsigned g = 0; g < ctrl->n_nasm; g++) {
        const NasmDev G = nasms[g];
        for (unsigned i = t0; i < G.n_init; i += stride) queue[G.queue_base + i] = G.init_ready[i] + G.tile_base + 1u;
    }
}

template <bool TENSOR_CORES>
__device__ __forceinline__ void run_tile(const LayerDev &L, const TileDev &T, const NasmDev &G, unsigned char *stage_mem, tc::Shared *sh,
                                         tc::PipeState &ps, CtrlDev *ctrl, StatusHost *status) {
    const unsigned tid = threadIdx.x;
    switch (L.type) {
        case CONV_LAYER: case FC_LAYER: case MATMUL_LAYER: case K_ATTENTION_LAYER: case V_ATTENTION_LAYER:
            if (TENSOR_CORES) tc::tile_gemm(L, T, G, stage_mem, sh, ps, ctrl, status);
            else if (tid < tc::NW) tile_gemm_ffma(L, T, tid, tc::NW);
            break;
        case RESIDUAL_LAYER: if (tid < tc::NW) tile_residual(L, T, tid, tc::NW); break;
        case MAXPOOL_LAYER: if (tid < tc::NW) tile_pool<true>(L, T, tid, tc::NW); break;
        case AVGPOOL_LAYER: if (tid < tc::NW) tile_pool<false>(L, T, tid, tc::NW); break;
        case LAYERNORM_LAYER: if (tid < tc::NW) tile_layernorm(L, T, tid, tc::NW); break;
        case SOFTMAX_LAYER: if (tid < tc::NW) tile_softmax(L, T, tid, tc::NW); break;
        case YOLO_LAYER: if (tid < tc::NW) tile_yolo(L, T, tid, tc::NW); break;
        case APPEND_LAYER: if (tid < tc::NW) tile_append(L, T, tid, tc::NW); break;
        default: break;
    }
}

template <bool TENSOR_CORES>
__global__ void __launch_bounds__(tc::NTHREADS, 1)
scheduler_kernel(const NasmDev *nasms, CtrlDev *ctrl, unsigned *queue, StatusHost *status, unsigned long long *prof) {
    extern __shared__ unsigned char smem_raw[];
    // stage buffers need 1024-byte alignment for the 128-byte swizzle
    unsigned char *stage_mem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    tc::Shared *sh = reinterpret_cast<tc::Shared *>(stage_mem + (TENSOR_CORES ? tc::STAGES * tc::STAGE_BYTES + tc::EPI_BYTES : 0u));
    const unsigned tid = threadIdx.x, warp = tid >> 5;
    const unsigned ctrl_warp = tc::NW >> 5;
    tc::PipeState ps;

    if (TENSOR_CORES) {
        if (tid == 0) {
            for (int s = 0; s < tc::STAGES; s++) { tc::mbar_init(&sh->full[s], tc::NW); tc::mbar_init(&sh->empty[s], 1u); tc::mbar_init(&sh->landed[s], 1u); }
            tc::mbar_init(&sh->accum, 1u);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            tc::fence_proxy_async_smem();
        }
        if (warp == ctrl_warp + 1u) tc::tmem_alloc(&sh->tmem_base, tc::TMEM_COLS);
        tc::tc_fence_before();
    }
    __syncthreads();
    if (TENSOR_CORES) tc::tc_fence_after();

    const unsigned n_nasm = ctrl->n_nasm;
    unsigned next = ASPEN_TILE_NONE;
    // Optional time accounting (per CTA, by the control thread): [0] waiting for a ready tile,
    // [1] completion + child update, [2 + layer] running tiles of that layer (index modulo PROF_LAYERS),
    // [2 + PROF_LAYERS + layer] tile counts.
    unsigned long long *my_prof = prof ? prof + (size_t)blockIdx.x * PROF_SLOTS : nullptr;
    unsigned long long t_mark = my_prof ? global_ns() : 0ull;
    while (true) {
        if (tid == tc::TMA_THREAD) {
            sh->tile = next != ASPEN_TILE_NONE ? next : pop_ready(ctrl, queue, status);
            if (my_prof) { unsigned long long now = global_ns(); my_prof[0] += now - t_mark; t_mark = now; }
        }
        __syncthreads();
        const unsigned gid = sh->tile;
        if (gid == ASPEN_TILE_NONE) break;
        unsigned g = 0;
        while (g + 1u < n_nasm && gid >= nasms[g + 1u].tile_base) g++;
        const NasmDev &G = nasms[g];
        const unsigned local = gid - G.tile_base;
        const TileDev T = G.tiles[local];
        const LayerDev &L = G.layers[T.layer];
        run_tile<TENSOR_CORES>(L, T, G, stage_mem, sh, ps, ctrl, status);
        __syncthreads();                                  // every thread's stores of this tile are issued
        if (warp == ctrl_warp) {
            if (my_prof && tid == tc::TMA_THREAD) {
                unsigned long long now = global_ns();
                my_prof[2 + T.layer % PROF_LAYERS] += now - t_mark; my_prof[2 + PROF_LAYERS + T.layer % PROF_LAYERS] += 1ull; t_mark = now;
            }
            next = ASPEN_TILE_NONE;
            if (!ps.dead && !sched::ld_relaxed(&ctrl->abort)) next = complete_tile(G, local, ctrl, queue, status);
            if (my_prof && tid == tc::TMA_THREAD) { unsigned long long now = global_ns(); my_prof[1] += now - t_mark; t_mark = now; }
        }
    }

    if (TENSOR_CORES) {
        tc::tc_fence_before();
        __syncthreads();
        if (warp == ctrl_warp + 1u) { tc::tc_fence_after(); tc::tmem_dealloc(sh->tmem_base, tc::TMEM_COLS); }
    }
}

}  // namespace sched
