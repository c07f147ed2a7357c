// Host side of the ready-pool / scheduling-engine API.  In the reference an rpool is a set of
// mutex-guarded queues and a dse is a pthread (src/rpool.c, src/dse.c); here the pool is the list
// of tile graphs whose device images are armed, and a dse group owns one CUDA stream plus the
// persistent scheduler kernel that drains every armed graph (engine.cu).
#include "internal.h"

#include <fstream>

// -1: not set by the program.  A caller that cannot be changed (a program written against the reference's
// header) picks the mode with the environment: ASPEN_B200_PRECISION=fp32 (or 1) selects the FFMA validation mode.
static thread_local int g_precision = -1;

extern "C" void aspen_b200_set_precision(int mode) { g_precision = mode ? 1 : 0; }

static int effective_precision() {
    if (g_precision >= 0) return g_precision;
    const char *v = getenv("ASPEN_B200_PRECISION");
    return (v && (!strcmp(v, "fp32") || !strcmp(v, "1"))) ? 1 : 0;
}

// ---- rpool -----------------------------------------------------------------------------------
extern "C" rpool_t *rpool_init(void) { return new rpool_t(); }

extern "C" void rpool_destroy(rpool_t *rpool) {
    if (!rpool) return;
    if (rpool->ref_dses.load() > 0) {
        ASPEN_ERR("ERROR: rpool_destroy: rpool is still referenced by %d dses.\n", rpool->ref_dses.load());
        return;
    }
    for (nasm_t *n : rpool->nasms) n->rpool = nullptr;
    delete rpool;
}

static size_t input_elements(const nasm_t *nasm) {
    const nasm_ldata_t &l0 = nasm->ldata[0];
    return (size_t)l0.out_mat_dims[OUT_H] * l0.out_mat_dims[OUT_W];
}

extern "C" void rpool_add_nasm_raw_input(rpool_t *rpool, nasm_t *nasm, void *input_data) {
    if (!rpool) { ASPEN_ERR("ERROR: rpool_add_nasm_raw_input: rpool is NULL.\n"); return; }
    if (!nasm) { ASPEN_ERR("ERROR: rpool_add_nasm_raw_input: nasm is NULL.\n"); return; }
    if (!nasm->has_graph) { ASPEN_ERR("ERROR: rpool_add_nasm_raw_input: nasm has no dependency graph.\n"); return; }
    if (nasm->rpool && nasm->rpool != rpool) { ASPEN_ERR("ERROR: rpool_add_nasm_raw_input: nasm already belongs to another rpool.\n"); return; }
    bool present = false;
    for (nasm_t *n : rpool->nasms) present |= n == nasm;
    if (!present) rpool->nasms.push_back(nasm);
    nasm->rpool = rpool;
    nasm->completed.store(0);
    // The device image needs an engine (device + stream).  If the pool is not served by a dse
    // group yet, the input is staged on the host and uploaded by dse_group_set_rpool.
    if (rpool->engine) {
        if (engine_attach_nasm(rpool->engine, nasm, input_data) != 0) ASPEN_ERR("ERROR: rpool_add_nasm_raw_input: device upload failed.\n");
    } else {
        nasm->staged_input.clear();
        if (input_data) nasm->staged_input.assign((const float *)input_data, (const float *)input_data + input_elements(nasm));
        nasm->staged = true;
    }
}

// Token-id input of a transformer (no counterpart in the reference, whose cfgs start at the hidden states).
extern "C" int aspen_b200_dnn_set_embedding(aspen_dnn_t *dnn, const float *token_table, unsigned int vocab, const float *position_table,
                                            unsigned int max_pos) {
    if (!dnn || !token_table || vocab == 0) { ASPEN_ERR("ERROR: aspen_b200_dnn_set_embedding: NULL dnn / table or empty vocabulary.\n"); return -1; }
    const unsigned int width = dnn->layers.empty() ? 0 : dnn->layers[0].params[MAT_M];
    if (width == 0) { ASPEN_ERR("ERROR: aspen_b200_dnn_set_embedding: the first layer of dnn \"%s\" has no hidden width (M).\n", dnn->name); return -1; }
    for (DeviceDnn *dd : dnn->dev)
        if (dd) { ASPEN_ERR("ERROR: aspen_b200_dnn_set_embedding: set the tables before the dnn's first graph is uploaded.\n"); return -1; }
    dnn->emb_token.assign(token_table, token_table + (size_t)vocab * width);
    dnn->emb_position.clear();
    if (position_table && max_pos) dnn->emb_position.assign(position_table, position_table + (size_t)max_pos * width);
    dnn->emb_vocab = vocab; dnn->emb_max_pos = position_table ? max_pos : 0; dnn->emb_width = width;
    return 0;
}

extern "C" void aspen_b200_rpool_add_nasm_tokens(rpool_t *rpool, nasm_t *nasm, const int *token_ids) {
    if (!rpool || !nasm || !token_ids) { ASPEN_ERR("ERROR: aspen_b200_rpool_add_nasm_tokens: NULL argument.\n"); return; }
    if (!rpool->engine) { ASPEN_ERR("ERROR: aspen_b200_rpool_add_nasm_tokens: attach the rpool to a dse group first (the gather runs on its device).\n"); return; }
    if (engine_in_service(rpool->engine)) {
        if (!nasm->has_graph) { ASPEN_ERR("ERROR: aspen_b200_rpool_add_nasm_tokens: nasm has no dependency graph.\n"); return; }
        if (nasm->rpool && nasm->rpool != rpool) { ASPEN_ERR("ERROR: aspen_b200_rpool_add_nasm_tokens: nasm already belongs to another rpool.\n"); return; }
        bool present = false;
        for (nasm_t *n : rpool->nasms) present |= n == nasm;
        if (!present) rpool->nasms.push_back(nasm);
        nasm->rpool = rpool;
        nasm->completed.store(0);
        if (engine_service_tokens(rpool->engine, nasm, token_ids) != 0) ASPEN_ERR("ERROR: aspen_b200_rpool_add_nasm_tokens: device upload failed.\n");
        return;
    }
    // the graph joins the pool exactly as with a raw input (image built on first use); layer 0 is then filled from the ids
    if (!nasm->dev || nasm->rpool != rpool) {
        rpool_add_nasm_raw_input(rpool, nasm, nullptr);
        if (!nasm->dev) return;
    } else {
        nasm->completed.store(0);
        if (engine_rearm(rpool->engine, nasm) != 0) return;
    }
    if (engine_set_tokens(nasm, token_ids) != 0) ASPEN_ERR("ERROR: aspen_b200_rpool_add_nasm_tokens: device gather failed.\n");
}

extern "C" void rpool_add_nasm(rpool_t *rpool, nasm_t *nasm, char *input_filename) {
    if (!rpool || !nasm) { ASPEN_ERR("ERROR: rpool_add_nasm: NULL argument.\n"); return; }
    const aspen_layer_t &first = nasm->dnn->layers[0];
    const unsigned int *p = first.params;
    size_t n = input_elements(nasm);
    std::vector<float> file(n, 0.f), data(n, 0.f);
    if (input_filename) {
        FILE *fp = fopen(input_filename, "rb");
        if (!fp) { ASPEN_ERR("ERROR: rpool_add_nasm: cannot open %s\n", input_filename); return; }
        size_t got = fread(file.data(), sizeof(float), n, fp);
        fclose(fp);
        if (got != n) ASPEN_ERR("ERROR: rpool_add_nasm: %s holds %zu of %zu values\n", input_filename, got, n);
    }
    if (p[OUT_C] != 0 && p[OUT_H] != 0 && p[OUT_W] != 0 && nasm->tr_seq_len == 0) {
        // file is NCHW, the pool wants NHWC (ref src/apu.c:638-664)
        const size_t C = p[OUT_C], H = p[OUT_H], W = p[OUT_W];
        for (size_t b = 0; b < nasm->batch_size; b++)
            for (size_t c = 0; c < C; c++)
                for (size_t h = 0; h < H; h++)
                    for (size_t w = 0; w < W; w++) data[((b * H + h) * W + w) * C + c] = file[((b * C + c) * H + h) * W + w];
    } else if (p[MAT_M] != 0) {
        data = file;
    } else {
        ASPEN_ERR("ERROR: rpool_add_nasm: first layer of dnn \"%s\" does not have output dimensions.\n", nasm->dnn->name);
        return;
    }
    rpool_add_nasm_raw_input(rpool, nasm, data.data());
}

extern "C" void rpool_reset_queue(rpool_t *rpool) {
    // Device queues are rebuilt when a graph is re-armed; nothing is pending between runs.
    if (!rpool) ASPEN_ERR("ERROR: rpool_reset_queue: rpool is NULL.\n");
}

extern "C" void apu_reset_nasm(nasm_t *nasm) {
    if (!nasm) return;
    nasm->completed.store(0);
    if (nasm->dev && nasm->rpool && nasm->rpool->engine) engine_rearm(nasm->rpool->engine, nasm);
}

extern "C" void rpool_reset_nasm(rpool_t *rpool, nasm_t *nasm) {
    if (!rpool || !nasm) { ASPEN_ERR("ERROR: rpool_reset_nasm: NULL argument.\n"); return; }
    if (nasm->rpool != rpool) { ASPEN_ERR("ERROR: rpool_reset_nasm: nasm \"%s_nasm_%d\" is not in rpool.\n", nasm->dnn->name, nasm->nasm_id); return; }
    apu_reset_nasm(nasm);   // keeps the input already resident in layer 0 (ref src/rpool.c:267-277)
}

// ---- dse group -------------------------------------------------------------------------------
extern "C" dse_group_t *dse_group_init(unsigned int num_dse) {
    dse_group_t *g = new dse_group_t();
    g->num_dses = num_dse;
    g->precision = effective_precision();
    g->device = engine_current_device();
    g->engine = engine_create(g->device, g->precision, num_dse);
    if (!g->engine) {
        ASPEN_ERR("ERROR: dse_group_init: no usable CUDA device / kernel image (sm_100a required).\n");
        delete g;
        return nullptr;
    }
    return g;
}

extern "C" void dse_group_set_rpool(dse_group_t *g, rpool_t *rpool) {
    if (!g) { ASPEN_ERR("ERROR: dse_group_set_rpool: dse_group is NULL\n"); return; }
    if (!rpool) { ASPEN_ERR("ERROR: dse_group_set_rpool: rpool is NULL\n"); return; }
    if (rpool->engine && rpool->engine != g->engine) { ASPEN_ERR("ERROR: dse_group_set_rpool: rpool is already served by another dse group\n"); return; }
    g->rpool = rpool;
    rpool->engine = g->engine;
    rpool->ref_dses.fetch_add(g->num_dses);
    for (nasm_t *n : rpool->nasms)
        if (n->staged) {
            if (engine_attach_nasm(g->engine, n, n->staged_input.empty() ? nullptr : n->staged_input.data()) != 0)
                ASPEN_ERR("ERROR: dse_group_set_rpool: device upload failed.\n");
            n->staged = false;
            n->staged_input.clear();
            n->staged_input.shrink_to_fit();
        }
}

extern "C" void dse_group_destroy(dse_group_t *g) {
    if (!g) return;
    engine_stop(g->engine);
    if (g->rpool) {
        g->rpool->ref_dses.fetch_sub(g->num_dses);
        for (nasm_t *n : g->rpool->nasms) engine_detach_nasm(n);
        g->rpool->engine = nullptr;
    }
    engine_destroy(g->engine);
    delete g;
}

extern "C" void dse_group_run(dse_group_t *g) {
    if (!g) { ASPEN_ERR("ERROR: dse_group_run: dse_group is NULL\n"); return; }
    if (!g->rpool) { ASPEN_ERR("ERROR: dse_group_run: no rpool set\n"); return; }
    if (engine_run(g->engine, g->rpool->nasms) != 0) ASPEN_ERR("ERROR: dse_group_run: launch failed\n");
}

extern "C" void dse_group_stop(dse_group_t *g) {
    if (!g) { ASPEN_ERR("ERROR: dse_group_stop: dse_group is NULL\n"); return; }
    engine_stop(g->engine);
}

extern "C" void dse_wait_for_nasm_completion(nasm_t *nasm) {
    if (!nasm) return;
    if (!nasm->dev) { ASPEN_ERR("ERROR: dse_wait_for_nasm_completion: nasm is not in a served rpool\n"); return; }
    if (engine_wait_nasm(nasm) != 0) ASPEN_ERR("ERROR: dse_wait_for_nasm_completion: nasm did not complete (engine status %d)\n",
                                               nasm->rpool && nasm->rpool->engine ? engine_status(nasm->rpool->engine) : -1);
}

extern "C" unsigned int dse_check_nasm_completion(nasm_t *nasm) {
    if (!nasm || !nasm->dev) return 0;
    return engine_poll_nasm(nasm);
}

extern "C" void dse_group_run_until_nasm_completion(dse_group_t *g, nasm_t *nasm) {
    dse_group_run(g);
    dse_wait_for_nasm_completion(nasm);
    dse_group_stop(g);
}

extern "C" int aspen_b200_dse_group_set_service(dse_group_t *g, int on) {
    if (!g) { ASPEN_ERR("ERROR: aspen_b200_dse_group_set_service: dse_group is NULL\n"); return -1; }
    return engine_set_service(g->engine, on);
}

extern "C" double aspen_b200_group_time_passes(dse_group_t *g, unsigned int warmup, unsigned int passes, unsigned long long *launches) {
    if (!g || !g->rpool) return -1.0;
    return engine_time_passes(g->engine, g->rpool->nasms, warmup, passes, launches);
}

extern "C" int aspen_b200_group_status(dse_group_t *g) { return g ? engine_status(g->engine) : ASPEN_B200_ERR_CUDA; }

extern "C" double aspen_b200_group_time_runs(dse_group_t *g, unsigned int warmup, unsigned int iters, unsigned long long *launches) {
    if (!g || !g->rpool) return -1.0;
    return engine_time_runs(g->engine, g->rpool->nasms, warmup, iters, launches);
}

extern "C" int aspen_b200_group_profile(dse_group_t *g, unsigned long long *out64, unsigned int *n_ctas) {
    return g ? engine_read_profile(g->engine, out64, n_ctas) : -1;
}

extern "C" void aspen_flush_dynamic_memory(void) { engine_flush(); }

extern "C" int aspen_b200_set_device(int device);   // engine.cu

// ---- results ---------------------------------------------------------------------------------
extern "C" long aspen_b200_nasm_get_ldata_packed(nasm_t *nasm, unsigned int idx, float *out) {
    if (!nasm || idx >= nasm->num_ldata || !out || !nasm->dev) return -1;
    return engine_read_ldata(nasm, idx, out);
}

// Native dim order of a layer's packed output (ref src/apu.c:248-283).
static int native_order(const nasm_ldata_t &ld, LAYER_PARAMS *order, unsigned int *dims) {
    const aspen_layer_t *l = ld.layer;
    const nasm_t *n = ld.nasm;
    memcpy(dims, l->params, sizeof(unsigned int) * NUM_PARAM_ELEMENTS);
    dims[BATCH] = n->batch_size;
    const LAYER_TYPE t = l->type;
    const bool img = t == CONV_LAYER || t == INPUT_LAYER || t == MAXPOOL_LAYER || t == AVGPOOL_LAYER || t == RESIDUAL_LAYER ||
                     t == APPEND_LAYER || t == YOLO_LAYER;
    if (img && l->params[MAT_M] == 0) { order[0] = BATCH; order[1] = OUT_H; order[2] = OUT_W; order[3] = OUT_C; return 4; }
    if (t == FC_LAYER || t == SOFTMAX_LAYER) { order[0] = BATCH; order[1] = OUT_C; return 2; }
    if (t == K_ATTENTION_LAYER) {
        dims[MAT_N] = n->tr_seq_len; dims[MAT_M] = n->tr_seq_len;
        order[0] = BATCH; order[1] = NUM_HEAD; order[2] = MAT_N; order[3] = MAT_M; return 4;
    }
    if (t == MATMUL_LAYER || t == LAYERNORM_LAYER || t == RESIDUAL_LAYER || t == INPUT_LAYER || t == V_ATTENTION_LAYER) {
        dims[MAT_N] = n->tr_seq_len;
        order[0] = BATCH; order[1] = MAT_N; order[2] = MAT_M; return 3;
    }
    return 0;
}

static ssize_t ldata_output(void **out_ptr, nasm_t *nasm, unsigned int idx, const LAYER_PARAMS *order) {
    const nasm_ldata_t &ld = nasm->ldata[idx];
    const size_t n = (size_t)ld.out_mat_dims[OUT_H] * ld.out_mat_dims[OUT_W];
    LAYER_PARAMS org[MAX_TENSOR_DIMS];
    unsigned int dims[NUM_PARAM_ELEMENTS];
    int nd = native_order(ld, org, dims);
    if (nd == 0) { ASPEN_ERR("Error in get_ldata_output: unsupported layer type.\n"); return -1; }
    size_t prod = 1;
    for (int i = 0; i < nd; i++) prod *= dims[org[i]];
    float *out = (float *)calloc(n ? n : 1, sizeof(float));
    bool same = order != nullptr && prod == n;
    for (int i = 0; same && i < nd; i++) same = order[i] == org[i];
    if (same || !order || prod != n) {
        // the wanted order is the one the device keeps: straight into the caller's buffer
        if (engine_read_ldata(nasm, idx, out) < 0) { free(out); return -1; }
        *out_ptr = out;
        return (ssize_t)(n * sizeof(float));
    }
    std::vector<float> packed(n);
    if (engine_read_ldata(nasm, idx, packed.data()) < 0) { free(out); return -1; }
    if (prod != n || !order) {
        memcpy(out, packed.data(), n * sizeof(float));   // shape not expressible: hand back native order
    } else {
        // destination strides per dim id, for the dims named by order[0..nd)
        size_t dst_stride[NUM_PARAM_ELEMENTS] = {};
        size_t s = 1;
        bool valid = true;
        for (int i = nd - 1; i >= 0; i--) {
            if (order[i] >= NUM_PARAM_ELEMENTS) { valid = false; break; }
            dst_stride[order[i]] = s;
            s *= dims[order[i]];
        }
        if (!valid || s != n) {
            memcpy(out, packed.data(), n * sizeof(float));
        } else {
            unsigned int pos[MAX_TENSOR_DIMS] = {};
            for (size_t i = 0; i < n; i++) {
                size_t d = 0;
                for (int k = 0; k < nd; k++) d += pos[k] * dst_stride[org[k]];
                out[d] = packed[i];
                for (int k = nd - 1; k >= 0; k--) {
                    if (++pos[k] < dims[org[k]]) break;
                    pos[k] = 0;
                }
            }
        }
    }
    *out_ptr = out;
    return (ssize_t)(n * sizeof(float));
}

extern "C" ssize_t dse_get_ldata_result(nasm_t *nasm, unsigned int ldata_idx, LAYER_PARAMS *order, void **out_ptr) {
    if (!nasm) { ASPEN_ERR("Error in get_ldata_output: ldata is NULL.\n"); return -1; }
    if (!out_ptr) { ASPEN_ERR("Error in get_ldata_output: out_ptr is NULL.\n"); return -1; }
    if (ldata_idx >= nasm->num_ldata || !nasm->dev) { ASPEN_ERR("Error in dse_get_ldata_result: no such layer output.\n"); return -1; }
    if (nasm->ldata[ldata_idx].layer->type != YOLO_LAYER) return ldata_output(out_ptr, nasm, ldata_idx, order);
    // Detection heads: per sample, the rows of every yolo layer one after the other (ref src/dse.c:476-511).
    std::vector<std::pair<float *, size_t>> parts;
    size_t total = 0;
    for (unsigned int i = 0; i < nasm->num_ldata; i++)
        if (nasm->ldata[i].layer->type == YOLO_LAYER) {
            void *d = nullptr;
            ssize_t sz = ldata_output(&d, nasm, i, order);
            if (sz < 0) { for (auto &pr : parts) free(pr.first); return -1; }
            parts.emplace_back((float *)d, (size_t)sz);
            total += (size_t)sz;
        }
    char *out = (char *)calloc(total ? total : 1, 1);
    size_t off = 0;
    for (unsigned int b = 0; b < nasm->batch_size; b++)
        for (auto &pr : parts) {
            size_t per = pr.second / nasm->batch_size;
            memcpy(out + off, (char *)pr.first + per * b, per);
            off += per;
        }
    for (auto &pr : parts) free(pr.first);
    *out_ptr = out;
    return (ssize_t)total;
}

extern "C" ssize_t dse_get_nasm_result(nasm_t *nasm, LAYER_PARAMS *order, void **out_ptr) {
    if (!nasm) { ASPEN_ERR("Error in dse_get_nasm_result: nasm is NULL.\n"); return -1; }
    return dse_get_ldata_result(nasm, nasm->num_ldata - 1, order, out_ptr);
}

// ---- tile-count search (ref src/apu_nasm.c:578-679) ------------------------------------------
static double time_nasm_ms(nasm_t *nasm, unsigned int iters) {
    rpool_t *rpool = rpool_init();
    dse_group_t *g = dse_group_init(0);
    if (!g) { rpool_destroy(rpool); return -1; }
    dse_group_set_rpool(g, rpool);
    rpool_add_nasm_raw_input(rpool, nasm, nullptr);
    double ms = aspen_b200_group_time_runs(g, 3, iters, nullptr);
    dse_group_destroy(g);
    nasm->rpool = nullptr;
    rpool_destroy(rpool);
    return ms < 0 ? -1 : ms / iters;
}

static nasm_t *generate(aspen_dnn_t *dnn, unsigned int batch, unsigned int seq, unsigned int num_iter) {
    auto make = [&](size_t n) { return seq ? apu_create_transformer_nasm(dnn, (unsigned int)n, batch, seq) : apu_create_nasm(dnn, (unsigned int)n, batch); };
    size_t num = 512, best_num = 512;
    nasm_t *nasm = make(num);
    if (!nasm) return nullptr;
    double t = time_nasm_ms(nasm, 20), best = t;
    if (t < 0) return nasm;   // no device: keep the first candidate
    for (unsigned int i = 0; i < num_iter; i++) {
        size_t old = num;
        if (t <= best * 1.05) num = (size_t)(num * 0.8);
        else num = (size_t)(num * 0.8 + best_num * 0.2);
        if (num < 1) num = 1;
        apu_destroy_nasm(nasm);
        nasm = make(num);
        t = time_nasm_ms(nasm, 20);
        if (t < best) { best = t; best_num = num; }
        if (num <= old * 1.10 && num >= old * 0.90) break;
    }
    apu_destroy_nasm(nasm);
    return make(best_num);
}

// Tile-shape search for this GPU: the reference tunes one number (tiles per layer) for its CPU kernels; here the
// candidates are tensor-core shaped quanta (rows x columns of whole MMA blocks) times a tile count per layer, each
// timed on the device with the scheduler kernel itself.  Values do not depend on the outcome.
extern "C" nasm_t *aspen_b200_generate_nasm(aspen_dnn_t *dnn, unsigned int batch_size, unsigned int seq_num, unsigned int *chosen) {
    if (!dnn || batch_size == 0) { ASPEN_ERR("aspen_b200_generate_nasm: no dnn or empty batch\n"); return nullptr; }
    static const unsigned int quanta[][2] = {{128, 128}, {256, 128}, {128, 256}};
    static const unsigned int counts[] = {100, 148, 180, 222, 296};
    const TileQuanta saved = g_quanta;
    double best = -1;
    unsigned int best_q = 0, best_n = counts[1];
    for (unsigned int q = 0; q < 3; q++)
        for (unsigned int n : counts) {
            aspen_b200_set_tile_quanta(quanta[q][0], quanta[q][1], saved.flop_per_ninst);
            nasm_t *cand = seq_num ? apu_create_transformer_nasm(dnn, n, batch_size, seq_num) : apu_create_nasm(dnn, n, batch_size);
            if (!cand) continue;
            const double t = time_nasm_ms(cand, 8);
            apu_destroy_nasm(cand);
            if (t > 0 && (best < 0 || t < best)) { best = t; best_q = q; best_n = n; }
        }
    aspen_b200_set_tile_quanta(quanta[best_q][0], quanta[best_q][1], saved.flop_per_ninst);
    nasm_t *out = seq_num ? apu_create_transformer_nasm(dnn, best_n, batch_size, seq_num) : apu_create_nasm(dnn, best_n, batch_size);
    g_quanta = saved;
    if (chosen) { chosen[0] = quanta[best_q][0]; chosen[1] = quanta[best_q][1]; chosen[2] = best_n; }
    return out;
}

extern "C" nasm_t *apu_generate_nasm(aspen_dnn_t *dnn, unsigned int batch_size, unsigned int num_iter) {
    return generate(dnn, batch_size, 0, num_iter);
}
extern "C" nasm_t *apu_generate_transformer_nasm(aspen_dnn_t *dnn, unsigned int batch_size, unsigned int seq_num, unsigned int num_iter) {
    return generate(dnn, batch_size, seq_num, num_iter);
}

// ---- print_* ---------------------------------------------------------------------------------
extern "C" void print_aspen_build_info(void) {
    printf("ASPEN B200 backend: sm_100a tile kernels + persistent device scheduler (built %s %s)\n", __DATE__, __TIME__);
}

extern "C" void print_tensor_info(aspen_tensor_t *t, int print_data) {
    if (!t) { printf("Error: Tensor is NULL.\n"); return; }
    printf("\t\tDims: ");
    for (unsigned int i = 0; i < t->num_dims; i++) printf("%s, ", param_type_str[t->data_dim_order[i]]);
    printf("\n\t\tSize: ");
    for (unsigned int i = 0; i < t->num_dims; i++) printf("%d, ", t->dims[t->data_dim_order[i]]);
    printf("\n\t\tNum Elements: %d\n\t\tElement Size: %d\n\t\tIs CPU data allocated? %s (%p)\n", t->num_elements, t->element_size,
           t->data ? "Yes" : "No", t->data);
    if (print_data && t->data) {
        unsigned int inner = t->num_dims ? t->dims[t->data_dim_order[t->num_dims - 1]] : 1;
        printf("\t\tData: ");
        for (unsigned int i = 0; i < t->num_elements; i++) {
            if (i % inner == 0) printf("\n\t\t\t%u: ", i / inner);
            printf("%3.3e ", ((float *)t->data)[i]);
        }
        printf("\n");
    }
}

extern "C" void print_layer_info(aspen_layer_t *l, int print_data) {
    if (!l) { printf("Error: Layer is NULL.\n"); return; }
    printf("//////// Printing Layer Info ////////\nLayer Index: %d\nLayer Type: %s\nLayer Activation: %s\nLayer Parents: ", l->layer_idx,
           layer_type_str[l->type], activation_type_str[l->activation]);
    for (int i = 0; i < NUM_PARENT_ELEMENTS; i++)
        if (l->parent_layers[i]) printf("%s: %d ", parent_type_str[i], l->parent_layers[i]->layer_idx);
    printf("\nLayer Params:\n");
    for (int i = 0; i < NUM_PARAM_ELEMENTS; i++)
        if (l->params[i] != 0) printf("\t%s: %d\n", param_type_str[i], l->params[i]);
    printf("Layer Tensors:\n");
    for (int i = 0; i < NUM_TENSORS; i++)
        if (l->tensors[i]) { printf("\t%s\n", tensor_type_str[i]); print_tensor_info(l->tensors[i], print_data); }
}

extern "C" void print_dnn_info(aspen_dnn_t *dnn, int print_data) {
    if (!dnn) { printf("Error: DNN is NULL.\n"); return; }
    printf("//////// Printing DNN Info ////////\nDNN Name: %s\nNumber of Layers: %d\n", dnn->name, dnn->num_layers);
    for (auto &l : dnn->layers) print_layer_info(&l, print_data);
    printf("//////// End of DNN Info ////////\n");
}

extern "C" void print_ninst_info(ninst_t *ni, int print_data) {
    if (!ni) { printf("Error: ninst is NULL.\n"); return; }
    printf("\t\tNinst Idx: %d\n\t\tState: %s\n\t\tNinst tile position: (H: %d, W: %d)\n\t\tNinst tile dims: (H: %d, W: %d)\n", ni->ninst_idx,
           ninst_state_str[ni->state], ni->out_mat_pos[OUT_H], ni->out_mat_pos[OUT_W], ni->tile_dims[OUT_H], ni->tile_dims[OUT_W]);
    printf("\t\tParent ninst (%zu): ", ni->parent_ninst_idx.size());
    for (unsigned int v : ni->parent_ninst_idx) printf("%d ", v);
    printf("\n\t\tChild ninst (%zu): ", ni->child_ninst_idx.size());
    for (unsigned int v : ni->child_ninst_idx) printf("%d ", v);
    printf("\n");
    if (print_data && ni->ldata->nasm->dev) {
        nasm_t *nasm = ni->ldata->nasm;
        unsigned int lidx = (unsigned int)(ni->ldata - nasm->ldata.data());
        std::vector<float> packed((size_t)ni->ldata->out_mat_dims[OUT_H] * ni->ldata->out_mat_dims[OUT_W]);
        if (engine_read_ldata(nasm, lidx, packed.data()) >= 0) {
            printf("\t\tData:");
            for (unsigned int w = 0; w < ni->tile_dims[OUT_W]; w++) {
                printf("\n\t\t\tN %d: ", w);
                for (unsigned int h = 0; h < ni->tile_dims[OUT_H]; h++)
                    printf("%3.3e ", packed[(size_t)(ni->out_mat_pos[OUT_W] + w) * ni->ldata->out_mat_dims[OUT_H] + ni->out_mat_pos[OUT_H] + h]);
            }
            printf("\n");
        }
    }
}

extern "C" void print_ldata_info(nasm_ldata_t *ld, int print_ninst, int print_data) {
    if (!ld) { printf("Error: ldata is NULL.\n"); return; }
    printf("//////////////////////// Printing ldata Info ////////////////////////\nOriginal layer index: %d\nOriginal layer type: %s\n",
           ld->layer->layer_idx, layer_type_str[ld->layer->type]);
    printf("Ldata Parents: ");
    for (int i = 0; i < NUM_PARENT_ELEMENTS; i++)
        if (ld->parent_ldata_idx_arr[i] != (unsigned int)-1) printf("%s: %d ", parent_type_str[i], ld->parent_ldata_idx_arr[i]);
    printf("\nLdata Children (%d): ", ld->num_child_ldata);
    for (unsigned int c : ld->child_ldata_idx) printf("%d ", c);
    printf("\nLdata flop per output element: %d\nLdata output matrix stride: %d\nLdata output matrix dimensions: (H: %d, W: %d)\n",
           ld->flop_per_output, ld->out_mat_stride, ld->out_mat_dims[OUT_H], ld->out_mat_dims[OUT_W]);
    printf("Ldata ninst tile dimensions: (H: %d, W: %d)\nNumber of ninst: %d\n", ld->ninst_tile_dims[OUT_H], ld->ninst_tile_dims[OUT_W], ld->num_ninst);
    if (print_ninst)
        for (unsigned int i = 0; i < ld->num_ninst; i++) {
            printf("\tNinst %d:\n", i);
            print_ninst_info(&ld->nasm->ninst[ld->ninst_start + i], print_data);
        }
}

extern "C" void print_nasm_info(nasm_t *nasm, int print_ninst, int print_data) {
    if (!nasm) { printf("Error: NASM is NULL.\n"); return; }
    printf("//////////////////////// Printing NASM Info ////////////////////////\nOriginal DNN name: %s\nNasm ID: %d\nNumber of ldata: %d\n",
           nasm->dnn->name, nasm->nasm_id, nasm->num_ldata);
    printf("Number of batch: %d\nNumber of ninst: %d\nFLOPs per ninst: %d\nTotal FLOPs: %ld\n", nasm->batch_size, nasm->num_ninst,
           nasm->flop_per_ninst, (long)nasm->total_flops);
    for (auto &ld : nasm->ldata) print_ldata_info(&ld, print_ninst, print_data);
    printf("//////////////////////// End of NASM Info ////////////////////////\n");
}

extern "C" void print_rpool_queue_info(rpool_queue_t *) { printf("Ready queues live on the device in this backend; see print_rpool_info.\n"); }
extern "C" void print_rpool_queue_group_info(rpool_queue_group_t *) { printf("Ready queues live on the device in this backend; see print_rpool_info.\n"); }
extern "C" void print_rpool_info(rpool_t *rpool) {
    if (!rpool) { printf("Error: rpool is NULL.\n"); return; }
    printf("//////////////////////// Printing Ready Pool Info ////////////////////////\nNumber of ref. DSEs: %d\nNumber of nasms: %zu\n",
           rpool->ref_dses.load(), rpool->nasms.size());
    for (nasm_t *n : rpool->nasms)
        printf("\tnasm %d (%s): %d tiles, on device: %s, completed: %d\n", n->nasm_id, n->dnn->name, n->num_ninst, n->dev ? "yes" : "no", dse_check_nasm_completion(n));
}
