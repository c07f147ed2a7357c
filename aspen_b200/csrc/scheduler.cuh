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
// The queue is a ticket ring: every tile is pushed at most once per run (per pass in service mode,
// where the ring holds a fixed number of passes and the kernel is launched again when they are used
// up), so it never wraps; slot value = global tile id + 1, 0 = not yet filled.  A popper that holds a
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
constexpr unsigned PROF_SLOTS = 2 + 2 * PROF_LAYERS + 2;

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

// Child update of a completed tile; called by the whole (converged) scheduler warp.  `children` holds
// (child tile, count the child waits for) pairs so one load feeds both the atomic and the test.
// Returns the global id of a child this CTA should run next (only when want_keep), or ASPEN_TILE_NONE.
// SERVICE: the counters are never reset between the passes of a graph; a pass only starts when the previous one is complete,
// so a child is ready whenever its counter reaches a multiple of the count it waits for.
template <bool SERVICE>
static __device__ unsigned complete_children(const NasmDev &G, unsigned child_off, unsigned child_cnt, CtrlDev *ctrl, unsigned *queue, bool want_keep) {
    const unsigned lane = threadIdx.x & 31u;
    const uint2 *edges = reinterpret_cast<const uint2 *>(G.children);
    __threadfence();                                     // release: this tile's output
    unsigned next = ASPEN_TILE_NONE;
    for (unsigned base = 0; base < child_cnt; base += 32u) {
        const unsigned idx = base + lane;
        unsigned child = ASPEN_TILE_NONE;
        bool ready = false;
        if (idx < child_cnt) {
            const uint2 e = edges[child_off + idx];
            child = e.x;
            const unsigned now = atomicAdd(&G.dep[child], 1u) + 1u;
            ready = SERVICE ? (now % e.y == 0u) : (now == e.y);
        }
        unsigned mask = __ballot_sync(0xffffffffu, ready);
        if (mask == 0u) continue;
        __threadfence();                                 // acquire the other parents' outputs (through the counters), then publish
        if (want_keep && next == ASPEN_TILE_NONE) {
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
    return next;
}

// Completion accounting (ref src/dse.c:80-106): layer counter -> layers-completed counter -> the
// graph's completed flag; run-wide tile count.  Not on the path of the next tile: done after it is posted.
static __device__ void complete_accounting(const NasmDev &G, unsigned layer, CtrlDev *ctrl, StatusHost *status) {
    if ((threadIdx.x & 31u) != 0u) return;
    unsigned d = atomicAdd(&G.layer_done[layer], 1u);
    unsigned t = atomicAdd(&ctrl->done, 1u);
    if (d + 1u == G.layer_tiles[layer]) {
        unsigned l = atomicAdd(G.layers_completed, 1u);
        if (l + 1u == G.n_layers) {
            __threadfence_system();
            *G.completed = 1u;                           // mapped host flag: the nasm is complete
        }
    }
    if (((t + 1u) & 1023u) == 0u || t + 1u == ctrl->total) status->tiles_done = t + 1u;
}

// ---- service mode ------------------------------------------------------------------------------
// The kernel stays resident while the host keeps asking for passes of the graphs it was launched with (the counterpart
// of the reference's DSE threads, which run from dse_group_run to dse_group_stop and serve whatever rpool_add_nasm
// brings, ref src/dse.c:20-108, 215-232).  The host asks for pass number p of a graph by writing p to the graph's
// SVC_TARGET word (a 4-byte copy that follows the input upload on the transfer stream).  An idle scheduler warp that
// finds an idle graph with target != started claims it (CAS on SVC_IDLE) and pushes its layer-0 tiles; those tiles
// prepare the input, everything else follows from the dependency counters.  The warp that retires the last tile of a
// pass writes the pass number to the graph's mapped host word and marks the graph idle.  The kernel leaves -- without
// error -- when no pass is running or asked for and the host has asked it to stop, when nothing has run for idle_ns,
// or when the queue of this launch is used up; the host launches it again if work is left.
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Looks at every graph; starts the next pass where one is asked for.  Whole (converged) warp.
// Returns bit 0: some graph has a pass in progress, bit 1: a pass is asked for but this launch's queue has no room left,
// bit 2: this warp started a pass.
static __device__ unsigned svc_scan(const NasmDev *nasms, unsigned n_nasm, CtrlDev *ctrl, unsigned *queue) {
    const unsigned lane = threadIdx.x & 31u;
    unsigned st = 0;
    for (unsigned g = 0; g < n_nasm; g++) {
        const NasmDev &G = nasms[g];
        unsigned go = 0;
        if (lane == 0) {
            if (ld_acquire(&G.svc[SVC_IDLE]) == 0u) go = 1u;
            else if (ld_acquire_sys(&G.svc[SVC_TARGET]) != ld_relaxed(&G.svc[SVC_STARTED])) {
                if (ld_relaxed(&ctrl->tail) + ctrl->total > ctrl->cap) go = 2u;
                else if (atomicCAS(&G.svc[SVC_IDLE], 1u, 0u) == 1u) {
                    // only the holder of the claim changes SVC_STARTED: look again now that it is ours
                    const unsigned started = ld_relaxed(&G.svc[SVC_STARTED]);
                    if (ld_acquire_sys(&G.svc[SVC_TARGET]) != started) {
                        asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(&G.svc[SVC_STARTED]), "r"(started + 1u) : "memory");
                        atomicAdd(&ctrl->busy, 1u);
                        go = 4u;
                    } else asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&G.svc[SVC_IDLE]), "r"(1u) : "memory");
                } else go = 1u;
            }
        }
        go = __shfl_sync(0xffffffffu, go, 0);
        st |= go;
        if (go == 4u) {
            unsigned pos = 0;
            if (lane == 0) pos = atomicAdd(&ctrl->tail, G.n_input);
            pos = __shfl_sync(0xffffffffu, pos, 0);
            for (unsigned i = lane; i < G.n_input; i += 32u)
                if (pos + i < ctrl->cap)
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&queue[pos + i]), "r"(i + G.tile_base + 1u) : "memory");
        }
    }
    return st;
}

// Completion accounting in service mode: one counter per graph; every n_exec-th completion ends a pass.
static __device__ void svc_account(const NasmDev *nasms, unsigned n_nasm, unsigned g, CtrlDev *ctrl, unsigned *queue) {
    const NasmDev &G = nasms[g];
    const unsigned lane = threadIdx.x & 31u;
    unsigned t = 0;
    if (lane == 0) { atomicAdd(&ctrl->done, 1u); t = atomicAdd(&G.svc[SVC_COUNT], 1u) + 1u; }
    t = __shfl_sync(0xffffffffu, t, 0);
    if (t % G.n_exec != 0u) return;
    if (lane == 0) {
        __threadfence_system();
        *G.completed = G.svc_base + t / G.n_exec;          // mapped host word: number of the pass that is complete
        __threadfence_system();
        atomicSub(&ctrl->busy, 1u);
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&G.svc[SVC_IDLE]), "r"(1u) : "memory");
    }
    __syncwarp();
    svc_scan(nasms, n_nasm, ctrl, queue);                  // the next pass of this graph may already be asked for
}

// Arms a service launch: empty queue, zero counters, every graph idle at the pass count the host has seen complete.
static __global__ void svc_arm_kernel(NasmDev *nasms, CtrlDev *ctrl, unsigned *queue, unsigned cap, unsigned total, unsigned long long stall_ns,
                               unsigned long long pipe_ns, unsigned long long idle_ns, unsigned svc_stop, unsigned svc_ahead) {
    const unsigned stride = gridDim.x * blockDim.x, t0 = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned n_nasm = ctrl->n_nasm;
    for (unsigned i = t0; i < cap; i += stride) queue[i] = 0u;
    for (unsigned g = 0; g < n_nasm; g++) {
        const NasmDev G = nasms[g];
        for (unsigned i = t0; i < G.n_tiles; i += stride) G.dep[i] = 0u;
        if (t0 == 0) { G.svc[SVC_STARTED] = G.svc_base; G.svc[SVC_IDLE] = 1u; G.svc[SVC_COUNT] = 0u; }
    }
    if (t0 == 0) {
        ctrl->head = 0u; ctrl->tail = 0u; ctrl->done = 0u; ctrl->total = total; ctrl->cap = cap;
        ctrl->abort = 0u; ctrl->stop = 0u; ctrl->stall_ns = stall_ns; ctrl->pipe_ns = pipe_ns;
        ctrl->svc_stop = svc_stop; ctrl->svc_close = 0u; ctrl->busy = 0u; ctrl->idle_ns = idle_ns; ctrl->svc_ahead = svc_ahead;
    }
}

// Resets the counters of every graph in the run and seeds the queue with the tiles that only
// depend on input tiles (push_first_layer_to_rpool, ref src/dse.c:443-470).
static __global__ void arm_kernel(NasmDev *nasms, CtrlDev *ctrl, unsigned *queue, unsigned total, unsigned n_init_total,
                           unsigned n_input_total, unsigned long long stall_ns, unsigned long long pipe_ns, unsigned ahead) {
    const unsigned stride = gridDim.x * blockDim.x, t0 = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned n_nasm = ctrl->n_nasm;
    for (unsigned i = t0; i < total; i += stride) queue[i] = 0u;
    __threadfence();
    for (unsigned g = 0; g < n_nasm; g++) {
        const NasmDev G = nasms[g];
        for (unsigned i = t0; i < G.n_tiles; i += stride) G.dep[i] = G.dep_init[i];
        for (unsigned i = t0; i < G.n_layers; i += stride) G.layer_done[i] = G.layer_done_init[i];
        if (t0 == 0) { *G.layers_completed = G.layers_done_init; *G.completed = 0u; }
    }
    if (t0 == 0) {
        ctrl->head = 0u; ctrl->tail = n_init_total; ctrl->done = n_input_total; ctrl->total = total; ctrl->cap = total;
        ctrl->abort = 0u; ctrl->stop = 0u; ctrl->stall_ns = stall_ns; ctrl->pipe_ns = pipe_ns; ctrl->svc_ahead = ahead;
    }
}
// Second step of arming (after every slot was cleared): write the initial ready tiles.
static __global__ void seed_kernel(NasmDev *nasms, CtrlDev *ctrl, unsigned *queue) {
    const unsigned stride = gridDim.x * blockDim.x, t0 = blockIdx.x * blockDim.x + threadIdx.x;
    for (unsigned g = 0; g < ctrl->n_nasm; g++) {
        const NasmDev G = nasms[g];
        for (unsigned i = t0; i < G.n_init; i += stride) queue[G.queue_base + i] = G.init_ready[i] + G.tile_base + 1u;
    }
}

template <bool TENSOR_CORES, bool ATTENTION, bool SERVICE>
__device__ __forceinline__ void run_tile(const LayerDev &L, const TileDev &T, const NasmDev &G, unsigned char *stage_mem, tc::Shared *sh,
                                         tc::PipeState &ps, CtrlDev *ctrl, StatusHost *status) {
    const unsigned tid = threadIdx.x;
    switch (L.type) {
        case CONV_LAYER: case FC_LAYER: case MATMUL_LAYER: case K_ATTENTION_LAYER: case V_ATTENTION_LAYER:
            if (TENSOR_CORES && ATTENTION && L.att_fused) {
                tc::AttnArgs a;
                a.seq = L.seq; a.hd = L.hd; a.heads = L.heads; a.masked = L.masked; a.ldc = L.ldc; a.round_out = L.round_out;
                a.att_p_ld = L.att_p_ld; a.att_p_round = L.att_p_round; a.out = L.out; a.att_p_out = L.att_p_out;
                a.qmap = (const unsigned char *)G.wmaps + (size_t)L.att_qmap * 128;
                a.kmap = (const unsigned char *)G.wmaps + (size_t)L.att_kmap * 128;
                a.vmap = (const unsigned char *)G.wmaps + (size_t)L.wmap * 128;
                tc::AttnPipe ap;
                ap.att_tiles = ps.att_tiles; ap.att_groups = ps.att_groups; ap.dead = ps.dead;
                ps.dead = tc::tile_attention(a, T, stage_mem, sh, ap, ctrl, status);
                ps.att_tiles++;
                ps.att_groups += tc::attention_groups(L.seq, L.masked, T);
            } else if (TENSOR_CORES) tc::tile_gemm(L, T, G, stage_mem, sh, ps, ctrl, status);
            else if (tid < tc::NW) tile_gemm_ffma(L, T, tid, tc::NW);
            break;
        case RESIDUAL_LAYER: if (tid < tc::NW) tile_residual(L, T, tid, tc::NW); break;
        case MAXPOOL_LAYER: if (tid < tc::NW) tile_pool<true>(L, T, tid, tc::NW); break;
        case AVGPOOL_LAYER: if (tid < tc::NW) tile_pool<false>(L, T, tid, tc::NW); break;
        case LAYERNORM_LAYER: if (tid < tc::NW) tile_layernorm(L, T, tid, tc::NW); break;
        case SOFTMAX_LAYER: if (tid < tc::NW) tile_softmax(L, T, tid, tc::NW); break;
        case YOLO_LAYER: if (tid < tc::NW) tile_yolo(L, T, tid, tc::NW); break;
        case APPEND_LAYER: if (tid < tc::NW) tile_append(L, T, tid, tc::NW); break;
        case INPUT_LAYER: if (SERVICE && tid < tc::NW) tile_input(G.input, L, T, tid, tc::NW); break;
        default: break;
    }
}

// ---- the persistent kernel -------------------------------------------------------------------
// Threads 0 .. tc::NTHREADS-1 are the EXECUTORS (worker warps, TMA thread, MMA thread): they run one tile
// after the other out of a two-slot mailbox in shared memory.  The last warp is the SCHEDULER: when
// the executors finish a tile it updates the children first (the first child that became ready is
// posted straight back to the executors), and does the completion accounting and the queue
// traffic while the executors already run the next tile.
//   mailbox[k], k = sequence number & 1:  scheduler writes the tile id, arrives on posted[k];
//   executors wait posted[k], run the tile, every executor thread arrives on finished[k];
//   the scheduler waits finished[k] (so all stores of the tile are ordered before its gpu-scope
//   fence and the counter updates), retires the tile and may then reuse slot k.
constexpr unsigned SCHED_THREADS = tc::NTHREADS + 32u;

// Executors' wait for the next tile.  The scheduler always posts an exit marker eventually (end of
// run, stop, stall, abort); the time bound only guards against that logic failing.
__device__ __forceinline__ bool wait_posted(unsigned long long *bar, unsigned parity, CtrlDev *ctrl, StatusHost *status) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns(), budget = 2ull * ctrl->stall_ns + 4ull * ctrl->pipe_ns + 1000000000ull;
    for (unsigned spin = 1;; spin++) {
        if (tc::mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            __nanosleep(64);
            if (global_ns() - t0 > budget) break;
        }
    }
    if (atomicCAS(&ctrl->abort, 0u, (unsigned)ASPEN_B200_ERR_PIPE) == 0u) {
        status->info0 = 7; status->info1 = blockIdx.x; status->status = ASPEN_B200_ERR_PIPE;
        __threadfence_system();
    }
    return false;
}

template <bool SERVICE>
static __device__ void scheduler_warp(const NasmDev *nasms, unsigned n_nasm, CtrlDev *ctrl, unsigned *queue, StatusHost *status,
                               tc::Shared *sh, unsigned long long *my_prof) {
    const unsigned lane = threadIdx.x & 31u;
    unsigned issued = 0, retired = 0;          // tiles posted to / retired from the mailbox
    unsigned fl_nasm[2] = {0, 0}, fl_off[2] = {0, 0}, fl_cnt[2] = {0, 0}, fl_layer[2] = {0, 0};   // tiles in flight
    unsigned acct_nasm = 0, acct_layer = ASPEN_TILE_NONE;   // completion accounting still to do
    unsigned next = ASPEN_TILE_NONE;           // a ready tile waiting for a free slot
    unsigned kept = ASPEN_TILE_NONE;           // a child made ready by a tile this CTA completed
    unsigned ticket = ASPEN_TILE_NONE;         // a queue position we hold and wait on
    bool closed = false;                        // no further tiles will be issued (end of run, stop, abort)
    bool no_tickets = false;                    // the queue has no unowned position left; kept children still run
    const unsigned total = ctrl->total, cap = ctrl->cap;
    unsigned last_done = 0;
    unsigned long long t_progress = __shfl_sync(0xffffffffu, global_ns(), 0), t_mark = t_progress;
    const unsigned long long window = ctrl->stall_ns;
    unsigned idle_spins = SERVICE ? 30u : 0u, turn = 0, flags = 0, done = 0, ahead_turn = 0;
    const unsigned ahead = ctrl->svc_ahead;   // service: the first idle turns already look for a pass to start
    while (true) {
        bool progressed = false;
        // control state is read by lane 0 and broadcast so the warp never diverges on it
        // (global loads cost an L2 round trip each: while tiles are in flight they are sampled every 8th turn)
        if (issued == retired || (turn++ & 7u) == 0u) {
            unsigned f = 0, d = 0;
            if (lane == 0) {
                f = (ld_relaxed(&ctrl->abort) != 0u ? 1u : 0u) | (ld_relaxed(&ctrl->stop) != 0u ? 2u : 0u);
                if (SERVICE && ld_relaxed(&ctrl->svc_close) != 0u) f |= 4u;
                d = ld_relaxed(&ctrl->done);
            }
            flags = __shfl_sync(0xffffffffu, f, 0);
            done = __shfl_sync(0xffffffffu, d, 0);
        }
        const bool halt = flags != 0u;
        // 1. retire the oldest tile in flight once every executor thread has finished it
        if (issued > retired) {
            const unsigned k = retired & 1u;
            unsigned ok = lane == 0 ? (unsigned)tc::mbar_test_wait(&sh->finished[k], (retired >> 1) & 1u) : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok) {
                if (my_prof && lane == 0) t_mark = global_ns();
                if (!(flags & 1u)) {
                    unsigned child = complete_children<SERVICE>(nasms[fl_nasm[k]], fl_off[k], fl_cnt[k], ctrl, queue, kept == ASPEN_TILE_NONE);
                    if (child != ASPEN_TILE_NONE) kept = child;
                    acct_nasm = fl_nasm[k]; acct_layer = fl_layer[k];
                }
                if (my_prof && lane == 0) my_prof[1] += global_ns() - t_mark;
                retired++;
                progressed = true;
            }
        }
        // 2. find the next tile
        if (halt) closed = true;
        if (!closed && next == ASPEN_TILE_NONE) {
            if (kept != ASPEN_TILE_NONE) { next = kept; kept = ASPEN_TILE_NONE; progressed = true; }
            else {
                // Only an idle CTA queues up for the next ready tile.  Claiming one while still busy was
                // measured to cost 40 % of throughput: the claimed tile waits in this CTA's mailbox while
                // other SMs that could have started it at once sit idle.
                bool take = ticket == ASPEN_TILE_NONE && !no_tickets && issued == retired;
                if (ahead != 0u && !take && ticket == ASPEN_TILE_NONE && !no_tickets && issued - retired == 1u && (ahead_turn++ & 15u) == 0u) {
                    // Busy with one tile, nothing lined up.  With several requests in the kernel the queue usually holds ready
                    // tiles that no idle CTA is waiting for: taking one now lets the executors go from this tile straight to
                    // the next while the completion (child counters, queue pushes) runs beside them.  Only with a backlog: a
                    // ticket held for a tile that is not there yet would keep that tile from an idle SM.
                    int backlog = 0;
                    if (lane == 0) backlog = (int)(ld_relaxed(&ctrl->tail) - ld_relaxed(&ctrl->head));
                    take = __shfl_sync(0xffffffffu, backlog, 0) >= (int)ahead;
                }
                if (take) {
                    unsigned t = lane == 0 ? atomicAdd(&ctrl->head, 1u) : 0u;
                    ticket = __shfl_sync(0xffffffffu, t, 0);
                    if (ticket >= cap) { ticket = ASPEN_TILE_NONE; no_tickets = true; }   // every tile that can be pushed has an owner
                }
                if (ticket != ASPEN_TILE_NONE) {
                    unsigned v = lane == 0 ? ld_acquire(&queue[ticket]) : 0u;
                    v = __shfl_sync(0xffffffffu, v, 0);
                    if (v != 0u) { next = v - 1u; ticket = ASPEN_TILE_NONE; progressed = true; }
                }
            }
        }
        // 3. post it when a mailbox slot is free
        if (next != ASPEN_TILE_NONE && issued - retired < 2u) {
            unsigned g = 0;
            while (g + 1u < n_nasm && next >= nasms[g + 1u].tile_base) g++;
            const TileDev T = nasms[g].tiles[next - nasms[g].tile_base];
            if (T.flags & TILE_WRITTEN_BY_PARENTS) {
                // nothing to execute: the tiles it waited for wrote its values; it completes right here
                if (!(flags & 1u)) {
                    unsigned child = complete_children<SERVICE>(nasms[g], T.child_off, T.child_cnt, ctrl, queue, kept == ASPEN_TILE_NONE);
                    if (child != ASPEN_TILE_NONE) kept = child;
                    if (SERVICE) svc_account(nasms, n_nasm, g, ctrl, queue);
                    else complete_accounting(nasms[g], T.layer, ctrl, status);
                }
            } else {
                const unsigned k = issued & 1u;
                if (lane == 0) { sh->tile_desc[k] = T; sh->tile_nasm[k] = g; sh->mailbox[k] = next; tc::mbar_arrive(&sh->posted[k]); }
                // remember what retiring this tile will need (loaded now, off the critical path)
                fl_nasm[k] = g; fl_off[k] = T.child_off; fl_cnt[k] = T.child_cnt; fl_layer[k] = T.layer;
                issued++;
            }
            next = ASPEN_TILE_NONE;
            progressed = true;
        }
        if (acct_layer != ASPEN_TILE_NONE) {
            if (SERVICE) svc_account(nasms, n_nasm, acct_nasm, ctrl, queue);
            else complete_accounting(nasms[acct_nasm], acct_layer, ctrl, status);
            acct_layer = ASPEN_TILE_NONE;
        }
        // 4. end of run / stall detection
        if (!SERVICE && done >= total) closed = true;
        if (issued == retired) {
            if (closed && (next == ASPEN_TILE_NONE || halt)) break;
            if (no_tickets && next == ASPEN_TILE_NONE && kept == ASPEN_TILE_NONE && ticket == ASPEN_TILE_NONE) break;   // can never get work again
        }
        if (progressed || done != last_done) {
            unsigned long long now = lane == 0 ? global_ns() : 0ull;
            last_done = done; t_progress = __shfl_sync(0xffffffffu, now, 0); idle_spins = 0;
            continue;
        }
        if (((++idle_spins) & 31u) == 0u) {
            unsigned long long now = lane == 0 ? global_ns() : 0ull;
            now = __shfl_sync(0xffffffffu, now, 0);
            unsigned svc = 1u;
            if (SERVICE && issued == retired && !closed) {
                // an idle CTA looks for passes to start, and decides when the kernel has nothing left to wait for
                svc = svc_scan(nasms, n_nasm, ctrl, queue);
                if (svc & 4u) t_progress = now;
                else if (!(svc & 1u)) {
                    unsigned leave = (svc & 2u) ? 1u : 0u;
                    if (lane == 0 && !leave) leave = (ld_relaxed(&ctrl->svc_stop) != 0u || now - t_progress > ctrl->idle_ns) ? 1u : 0u;
                    leave = __shfl_sync(0xffffffffu, leave, 0);
                    if (leave) {
                        if (lane == 0) atomicExch(&ctrl->svc_close, 1u);
                        closed = true;
                    }
                }
            }
            if (now - t_progress > window && issued == retired && (svc & 1u)) {
                // nothing running here, nothing completed anywhere for a whole window: the graph cannot progress
                if (lane == 0 && atomicCAS(&ctrl->abort, 0u, (unsigned)ASPEN_B200_ERR_STALL) == 0u) {
                    status->info0 = ticket; status->info1 = done; status->status = ASPEN_B200_ERR_STALL;
                    __threadfence_system();
                }
                closed = true;
            }
            if (my_prof && lane == 0 && issued == retired) my_prof[0] += 1ull;   // idle polls with nothing in flight
        }
        __nanosleep(issued == retired ? 100u : 20u);
    }
    if (lane == 0) { sh->mailbox[issued & 1u] = ASPEN_TILE_NONE; tc::mbar_arrive(&sh->posted[issued & 1u]); }
}

// ATTENTION: the instantiation that contains the fused attention tile.  It is a kernel of its own because the mere presence
// of that code changes the register allocation of the contraction tile's main loop (measured: the whole kernel 40 % slower);
// graphs without a fused attention layer run the instantiation without it.
// SERVICE: the kernel serves pass after pass of its graphs until the host stops it (see "service mode" above).
template <bool TENSOR_CORES, bool ATTENTION = false, bool SERVICE = false>
__global__ void __launch_bounds__(SCHED_THREADS, 1)
scheduler_kernel(const NasmDev *nasms, CtrlDev *ctrl, unsigned *queue, StatusHost *status, unsigned long long *prof) {
    extern __shared__ unsigned char smem_raw[];
    // stage buffers need 1024-byte alignment for the 128-byte swizzle
    unsigned char *stage_mem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    tc::Shared *sh = reinterpret_cast<tc::Shared *>(stage_mem + (TENSOR_CORES ? tc::STAGES * tc::STAGE_BYTES + tc::EPI_BYTES + tc::RES_BYTES : 0u));
    const unsigned tid = threadIdx.x, warp = tid >> 5;
    const unsigned ctrl_warp = tc::NW >> 5;
    tc::PipeState ps;

    if (tid == 0) {
        for (int s = 0; s < tc::STAGES; s++) { tc::mbar_init(&sh->full[s], tc::NW); tc::mbar_init(&sh->empty[s], 1u); tc::mbar_init(&sh->landed[s], 1u); }
        tc::mbar_init(&sh->accum, 1u);
        for (unsigned w = 0; w < tc::NW / 32u; w++) tc::mbar_init(&sh->res_full[w], 1u);
        tc::mbar_init(&sh->att_q, 1u); tc::mbar_init(&sh->att_k, 1u); tc::mbar_init(&sh->att_v, 1u);
        tc::mbar_init(&sh->att_s, 1u); tc::mbar_init(&sh->att_p, tc::NW); tc::mbar_init(&sh->att_o, 1u);
        for (int k = 0; k < 2; k++) { tc::mbar_init(&sh->posted[k], 1u); tc::mbar_init(&sh->finished[k], tc::NTHREADS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::fence_proxy_async_smem();
    }
    if (TENSOR_CORES) {
        if (warp == ctrl_warp + 1u) tc::tmem_alloc(&sh->tmem_base, tc::TMEM_COLS);
        tc::tc_fence_before();
    }
    __syncthreads();
    if (TENSOR_CORES) tc::tc_fence_after();

    const unsigned n_nasm = ctrl->n_nasm;
    // Optional time accounting per CTA: [0] scheduler idle polls, [1] completion + child update (ns),
    // [2 + layer] ns the executors spent on tiles of that layer (index modulo PROF_LAYERS),
    // [2 + PROF_LAYERS + layer] tile counts, [PROF_SLOTS - 1] ns the executors waited for a tile.
    unsigned long long *my_prof = prof ? prof + (size_t)blockIdx.x * PROF_SLOTS : nullptr;

    if (warp == (SCHED_THREADS >> 5) - 1u) {
        scheduler_warp<SERVICE>(nasms, n_nasm, ctrl, queue, status, sh, my_prof);
    } else {
        unsigned long long t_mark = my_prof ? global_ns() : 0ull;
        for (unsigned seq = 0;; seq++) {
            const unsigned k = seq & 1u;
            if (!wait_posted(&sh->posted[k], (seq >> 1) & 1u, ctrl, status)) break;
            const unsigned gid = sh->mailbox[k];
            if (gid == ASPEN_TILE_NONE) break;
            if (my_prof && tid == 0) { unsigned long long now = global_ns(); my_prof[PROF_SLOTS - 1] += now - t_mark; t_mark = now; }
            const NasmDev &G = nasms[sh->tile_nasm[k]];
            const TileDev T = sh->tile_desc[k];
            const LayerDev &L = G.layers[T.layer];
            run_tile<TENSOR_CORES, ATTENTION, SERVICE>(L, T, G, stage_mem, sh, ps, ctrl, status);
            if (my_prof && tid == 0) {
                unsigned long long now = global_ns();
                my_prof[2 + T.layer % PROF_LAYERS] += now - t_mark; my_prof[2 + PROF_LAYERS + T.layer % PROF_LAYERS] += 1ull; t_mark = now;
            }
            tc::mbar_arrive(&sh->finished[k]);             // release (CTA scope): this thread's stores of the tile
        }
    }

    if (TENSOR_CORES) tc::tc_fence_before();
    __syncthreads();
    if (TENSOR_CORES && warp == ctrl_warp + 1u) { tc::tc_fence_after(); tc::tmem_dealloc(sh->tmem_base, tc::TMEM_COLS); }
}

}  // namespace sched
