// Tile dependency graph: which parent tiles each ninst reads, child lists, .nasm files.
//
// The reference finds parents by visiting every output element of a tile and every input element
// it touches, with a linear duplicate scan (ninst_find_parent, ref src/apu_nasm.c:49-466) -- tens of
// seconds per network.  Here each layer type enumerates only the positions at which the parent
// tile can change, in the reference's visiting order (tile column outer, tile row inner, then the
// per-type input loops), with O(1) duplicate detection, so the parent LISTS (order included, as
// written to .nasm files) come out identical in milliseconds.
#include "internal.h"

#include <unordered_set>

namespace {

struct ParentFinder {
    nasm_t *nasm;
    std::vector<unsigned int> stamp;     // stamp[tile] == cur  <=>  already listed for this ninst
    unsigned int cur = 0;
    std::vector<unsigned int> *list = nullptr;

    explicit ParentFinder(nasm_t *n) : nasm(n), stamp(n->num_ninst, 0) {}

    static unsigned int tile_of(const nasm_ldata_t &pl, unsigned int h, unsigned int w) {
        const unsigned int th = pl.ninst_tile_dims[OUT_H], tw = pl.ninst_tile_dims[OUT_W];
        const unsigned int per_col = (unsigned int)round_up(pl.out_mat_dims[OUT_H], th) / th;
        return pl.ninst_start + (w / tw) * per_col + h / th;
    }
    bool seen(unsigned int t) const { return stamp[t] == cur; }
    bool add(unsigned int t) {
        if (stamp[t] == cur) return false;
        stamp[t] = cur;
        list->push_back(t);
        return true;
    }
    unsigned int tile_from_tensor_pos(const nasm_ldata_t &pl, const unsigned int *tp) const {
        unsigned int mp[2];
        out_mat_pos_from_tensor_pos(&pl, tp, mp);
        return tile_of(pl, mp[OUT_H], mp[OUT_W]);
    }

    void run(ninst_t &ni, std::vector<unsigned int> &out, std::vector<unsigned int> &extra);
};

void ParentFinder::run(ninst_t &ni, std::vector<unsigned int> &out, std::vector<unsigned int> &extra) {
    nasm_ldata_t &ld = *ni.ldata;
    const aspen_layer_t *l = ld.layer;
    const unsigned int *p = l->params;
    const LAYER_TYPE type = l->type;
    if (type == INPUT_LAYER) return;
    cur++;
    list = &out;
    const nasm_ldata_t &p0 = nasm->ldata[ld.parent_ldata_idx_arr[PARENT_0]];
    const nasm_ldata_t *p1 = ld.parent_ldata_idx_arr[PARENT_1] != (unsigned int)-1 ? &nasm->ldata[ld.parent_ldata_idx_arr[PARENT_1]] : nullptr;
    const unsigned int seq = nasm->tr_seq_len, batch = nasm->batch_size;
    const unsigned int w0 = ni.out_mat_pos[OUT_W], h0 = ni.out_mat_pos[OUT_H];
    const unsigned int tw = ni.tile_dims[OUT_W], th = ni.tile_dims[OUT_H];
    const unsigned int p0th = p0.ninst_tile_dims[OUT_H], p0tw = p0.ninst_tile_dims[OUT_W];
    std::unordered_set<uint64_t> done;   // signatures of element visits that cannot add anything new
    uint64_t last_sig = ~0ull;

    for (unsigned int w = w0; w < w0 + tw; w++) {
        unsigned int mp[2];
        mp[OUT_W] = w;
        if (type == CONV_LAYER || type == MAXPOOL_LAYER || type == AVGPOOL_LAYER) {
            // Independent of the output row: the first row of each column lists everything.
            unsigned int tp[NUM_PARAM_ELEMENTS] = {}, ip[NUM_PARAM_ELEMENTS] = {};
            mp[OUT_H] = h0;
            tensor_pos_from_out_mat_pos(&ld, mp, tp);
            ip[BATCH] = tp[BATCH];
            if (ip[BATCH] >= batch) continue;
            for (unsigned int c = 0; c < p[IN_C]; c += p0th - c % p0th) {   // first channel of each parent row block
                ip[OUT_C] = c;
                for (unsigned int kh = 0; kh < p[WEIGHT_H]; kh++) {
                    ip[OUT_H] = tp[OUT_H] * p[STRIDE] + kh * p[DILATION] - p[PADDING];   // unsigned wrap == "negative"
                    if (ip[OUT_H] >= p[IN_H]) continue;
                    for (unsigned int kw = 0; kw < p[WEIGHT_W]; kw++) {
                        ip[OUT_W] = tp[OUT_W] * p[STRIDE] + kw * p[DILATION] - p[PADDING];
                        if (ip[OUT_W] >= p[IN_W]) continue;
                        add(tile_from_tensor_pos(p0, ip));
                    }
                }
            }
        } else if (type == FC_LAYER) {
            // Column = one sample; reads every channel and pixel of it.
            const unsigned int b = w;
            if (b >= batch) continue;
            for (unsigned int c = 0; c < p[IN_C]; c += p0th - c % p0th) {
                unsigned int last = (unsigned int)-1;
                for (unsigned int ih = 0; ih < p[IN_H]; ih++)
                    for (unsigned int iw = 0; iw < p[IN_W]; iw++) {
                        unsigned int ip[NUM_PARAM_ELEMENTS] = {};
                        ip[BATCH] = b; ip[OUT_C] = c; ip[OUT_H] = ih; ip[OUT_W] = iw;
                        unsigned int t = tile_from_tensor_pos(p0, ip);
                        if (t != last) { add(t); last = t; }
                    }
            }
        } else if (type == MATMUL_LAYER) {
            unsigned int tp[NUM_PARAM_ELEMENTS] = {};
            mp[OUT_H] = h0;
            tensor_pos_from_out_mat_pos(&ld, mp, tp);
            if (tp[BATCH] >= batch || tp[MAT_N] >= seq) continue;
            const unsigned int pm = p0.layer->params[MAT_M];
            for (unsigned int k = 0; k < p[MAT_K] && k < pm; k += p0th - k % p0th) {
                unsigned int ip[NUM_PARAM_ELEMENTS] = {};
                ip[BATCH] = tp[BATCH]; ip[MAT_M] = k; ip[MAT_N] = tp[MAT_N];
                add(tile_from_tensor_pos(p0, ip));
            }
        } else {
            // Element-wise dependent types: visit rows, skipping visits whose candidate list equals
            // that of an earlier visit (they can only produce duplicates).
            for (unsigned int h = h0; h < h0 + th; h++) {
                mp[OUT_H] = h;
                unsigned int tp[NUM_PARAM_ELEMENTS] = {}, ip[NUM_PARAM_ELEMENTS] = {};
                tensor_pos_from_out_mat_pos(&ld, mp, tp);
                ip[BATCH] = tp[BATCH];
                if (type == RESIDUAL_LAYER) {
                    if (p[MAT_M] == 0) { ip[OUT_C] = tp[OUT_C]; ip[OUT_H] = tp[OUT_H]; ip[OUT_W] = tp[OUT_W]; }
                    else { ip[MAT_M] = tp[MAT_M]; ip[MAT_N] = tp[MAT_N]; ip[OUT_C] = tp[OUT_C]; ip[OUT_H] = tp[OUT_H]; ip[OUT_W] = tp[OUT_W]; }
                    bool img_ok = ip[BATCH] < batch && ip[OUT_C] < p[IN_C] && ip[OUT_H] < p[IN_H] && ip[OUT_W] < p[IN_W];
                    bool mat_ok = ip[BATCH] < batch && ip[MAT_M] < p[MAT_M] && ip[MAT_N] < seq;
                    if (!(img_ok || mat_ok) || !p1) continue;
                    unsigned int t0 = tile_from_tensor_pos(p0, ip), t1 = tile_from_tensor_pos(*p1, ip);
                    const uint64_t sig = ((uint64_t)t0 << 32) | t1;
                    if (sig == last_sig || !done.insert(sig).second) continue;
                    last_sig = sig;
                    // The reference carries its duplicate flag from the first operand to the second
                    // (src/apu_nasm.c:118-151): the second operand's tile is listed only if the first
                    // operand's tile was new at this element.  Kept for graph/file identity; the true
                    // dependency is added to `extra` below.
                    bool dup = !add(t0);
                    if (seen(t1)) dup = true;
                    if (!dup) add(t1);
                } else if (type == SOFTMAX_LAYER) {
                    memcpy(ip, tp, sizeof ip);
                    if (!(ip[BATCH] < batch && ip[OUT_C] < p[IN_C] && ip[OUT_H] < p[IN_H] && ip[OUT_W] < p[IN_W])) continue;
                    add(tile_from_tensor_pos(p0, ip));
                } else if (type == YOLO_LAYER) {
                    unsigned int hw = p[IN_H] * p[IN_W];
                    unsigned int aidx = tp[OUT_W] / hw, rem = tp[OUT_W] % hw;
                    ip[OUT_H] = rem / p[IN_W]; ip[OUT_W] = rem % p[IN_W];
                    ip[OUT_C] = tp[OUT_C] + aidx * p[OUT_C];
                    if (!(ip[BATCH] < batch && ip[OUT_C] < p[IN_C] && ip[OUT_H] < p[IN_H] && ip[OUT_W] < p[IN_W])) continue;
                    add(tile_from_tensor_pos(p0, ip));
                } else if (type == APPEND_LAYER) {
                    const nasm_ldata_t *target;
                    if (tp[OUT_C] < p[IN_C]) {
                        target = &p0;
                        ip[OUT_C] = tp[OUT_C]; ip[OUT_W] = tp[OUT_W] / p[STRIDE]; ip[OUT_H] = tp[OUT_H] / p[STRIDE];
                    } else {
                        target = p1;
                        ip[OUT_C] = tp[OUT_C] - p[IN_C]; ip[OUT_W] = tp[OUT_W]; ip[OUT_H] = tp[OUT_H];
                    }
                    if (!target) continue;
                    if (!(ip[BATCH] < batch && ip[OUT_C] < p[IN_C] && ip[OUT_H] < p[IN_H] && ip[OUT_W] < p[IN_W])) continue;
                    add(tile_from_tensor_pos(*target, ip));
                } else if (type == LAYERNORM_LAYER) {
                    ip[MAT_M] = tp[MAT_M]; ip[MAT_N] = tp[MAT_N];
                    if (!(ip[BATCH] < batch && ip[MAT_M] < p0.layer->params[MAT_M] && ip[MAT_N] < seq)) continue;
                    add(tile_from_tensor_pos(p0, ip));
                } else if (type == K_ATTENTION_LAYER) {
                    // scores[key = row][query = column]: PARENT_0 holds the queries, PARENT_1 the keys
                    const unsigned int hd = p[NUM_HIDDEN] / p[NUM_HEAD], base = tp[NUM_HEAD] * hd;
                    const unsigned int q_tile_w = (tp[BATCH] * seq + tp[MAT_N]) / p0tw;
                    if (!p1) continue;
                    const unsigned int k_tile_w = (tp[BATCH] * seq + tp[MAT_M]) / p1->ninst_tile_dims[OUT_W];
                    const uint64_t sig = ((uint64_t)q_tile_w << 32) | k_tile_w;
                    if (sig == last_sig || !done.insert(sig).second) continue;
                    last_sig = sig;
                    for (unsigned int k = 0; k < p[MAT_K]; k++) {
                        ip[MAT_M] = k + base; ip[MAT_N] = tp[MAT_N];
                        if (ip[BATCH] < batch && ip[MAT_M] < p0.layer->params[MAT_M] && ip[MAT_N] < seq)
                            add(tile_from_tensor_pos(p0, ip));
                    }
                    for (unsigned int k = 0; k < p[MAT_K]; k++) {
                        ip[MAT_N] = tp[MAT_M]; ip[MAT_M] = k + base;
                        if (ip[BATCH] < batch && ip[MAT_M] < p1->layer->params[MAT_M] && ip[MAT_N] < seq)
                            add(tile_from_tensor_pos(*p1, ip));
                    }
                } else if (type == V_ATTENTION_LAYER) {
                    // out[feature = row][query = column] = sum_s P[s][(b, head, query)] * V[s][feature]
                    const unsigned int hd = p[NUM_HIDDEN] / p[NUM_HEAD], head = tp[MAT_M] / hd;
                    if (!p1) continue;
                    const unsigned int p_col = tp[BATCH] * seq * p0.layer->params[NUM_HEAD] + head * seq + tp[MAT_N];
                    const unsigned int v_row_tile = tp[MAT_M] / p1->ninst_tile_dims[OUT_H];
                    const uint64_t sig = ((uint64_t)(p_col / p0tw) << 32) | v_row_tile;
                    if (sig == last_sig || !done.insert(sig).second) continue;
                    last_sig = sig;
                    ip[NUM_HEAD] = head;
                    for (unsigned int k = 0; k < seq; k++) {
                        ip[MAT_M] = k; ip[MAT_N] = tp[MAT_N];
                        if (ip[BATCH] < batch && ip[MAT_M] < seq && ip[MAT_N] < seq && ip[NUM_HEAD] < p0.layer->params[NUM_HEAD])
                            add(tile_from_tensor_pos(p0, ip));
                    }
                    for (unsigned int k = 0; k < seq; k++) {
                        ip[MAT_N] = k; ip[MAT_M] = tp[MAT_M];
                        if (ip[BATCH] < batch && ip[MAT_M] < p1->layer->params[MAT_M] && ip[MAT_N] < seq)
                            add(tile_from_tensor_pos(*p1, ip));
                    }
                } else {
                    ASPEN_ERR("ERROR: Unsupported layer type %s in parent search\n", layer_type_str[type]);
                    return;
                }
            }
        }
    }

    // True data dependencies the reference's lists can miss (see the residual note above; its
    // softmax bounds test `1 < IN_H` never holds).  The device scheduler waits on list + extra.
    list = &extra;
    if (type == RESIDUAL_LAYER && p1) {
        for (unsigned int w = w0; w < w0 + tw; w++)
            for (unsigned int h = h0; h < h0 + th; h++) {
                add(tile_of(p0, h, w));
                add(tile_of(*p1, h, w));
            }
    } else if (type == SOFTMAX_LAYER) {
        for (unsigned int w = w0; w < w0 + tw; w++)
            for (unsigned int h = h0; h < h0 + th; h++) add(tile_of(p0, h, w));
    }
}

}  // namespace

void graph_find_parents(nasm_t *nasm) {
    ParentFinder pf(nasm);
    for (auto &ni : nasm->ninst) {
        ni.parent_ninst_idx.clear();
        ni.extra_parent_idx.clear();
        pf.run(ni, ni.parent_ninst_idx, ni.extra_parent_idx);
        if (ni.parent_ninst_idx.size() > MAX_PARENT_NINST_NUM) ASPEN_ERR("ninst %u has more than %d parents\n", ni.ninst_idx, MAX_PARENT_NINST_NUM);
    }
}

// Children in ascending tile order, as the reference's forward scan yields (src/apu_nasm.c:544-576).
void graph_set_children(nasm_t *nasm) {
    for (auto &ni : nasm->ninst) ni.child_ninst_idx.clear();
    for (auto &ni : nasm->ninst)
        for (unsigned int par : ni.parent_ninst_idx) nasm->ninst[par].child_ninst_idx.push_back(ni.ninst_idx);
    nasm->has_graph = true;
}

// ---- public: create / destroy / reset -------------------------------------------------------
static nasm_t *create_full(aspen_dnn_t *dnn, unsigned int min_ninst, unsigned int batch, unsigned int seq) {
    nasm_t *nasm = nasm_create_tiles(dnn, g_quanta.flop_per_ninst, batch, min_ninst, seq);
    if (!nasm) return nullptr;
    graph_find_parents(nasm);
    graph_set_children(nasm);
    return nasm;
}

extern "C" nasm_t *apu_create_nasm(aspen_dnn_t *dnn, unsigned int min_ninst_per_ldata, unsigned int batch_size) {
    return create_full(dnn, min_ninst_per_ldata, batch_size, 0);
}
extern "C" nasm_t *apu_create_transformer_nasm(aspen_dnn_t *dnn, unsigned int min_ninst_per_ldata, unsigned int batch_size, unsigned int seq_num) {
    return create_full(dnn, min_ninst_per_ldata, batch_size, seq_num);
}

extern "C" void apu_destroy_nasm(nasm_t *nasm) {
    if (!nasm) return;
    if (nasm->rpool) {
        auto &v = nasm->rpool->nasms;
        for (size_t i = 0; i < v.size(); i++)
            if (v[i] == nasm) { v.erase(v.begin() + i); break; }
    }
    engine_detach_nasm(nasm);
    nasm->dnn->ref_nasms.fetch_sub(1);
    delete nasm;
}

// ---- .nasm text files (ref src/apu_file_io.c:811-1094) ---------------------------------------
extern "C" void apu_save_nasm_to_file(nasm_t *nasm, char *filename) {
    if (!nasm) { ASPEN_ERR("ASPEN NASM to save is null.\n"); return; }
    if (!filename) { ASPEN_ERR("ASPEN NASM file name not specified.\n"); return; }
    FILE *fp = fopen(filename, "wb");
    if (!fp) { ASPEN_ERR("Error: apu_save_nasm_to_file Failed to open file %s for writing\n", filename); return; }
    fprintf(fp, "ASPEN_NASM\nDNN_NAME:%s\nNUM_BATCH:%d\nMIN_NINST_PER_LDATA:%d\nTOTAL_FLOPS:%ld\nFLOP_PER_NINST:%d\nSEQ_LEN:%d\nNASM_NINSTS:\n",
            nasm->dnn->name, nasm->batch_size, nasm->min_ninst_per_ldata, (long)nasm->total_flops, nasm->flop_per_ninst, nasm->tr_seq_len);
    for (auto &ni : nasm->ninst) {
        fprintf(fp, "\tNINST_IDX:%ld\n\tNUM_CHILD_NINSTS:%d\n\tNUM_PARENT_NINSTS:%d\n\tPARENT_NINSTS:\n", (long)ni.ninst_idx,
                (int)ni.child_ninst_idx.size(), (int)ni.parent_ninst_idx.size());
        for (size_t k = 0; k < ni.parent_ninst_idx.size(); k++) fprintf(fp, "\t\t%d %d\n", (int)k, ni.parent_ninst_idx[k]);
        fprintf(fp, "\tPARENT_NINSTS_END\n\tNUM_CHILD_NINSTS:%d\n\tCHILD_NINST_IDXES:\n", (int)ni.child_ninst_idx.size());
        for (size_t k = 0; k < ni.child_ninst_idx.size(); k++) fprintf(fp, "\t\t%d %ld\n", (int)k, (long)ni.child_ninst_idx[k]);
        fprintf(fp, "\tCHILD_NINST_IDXES_END\n\tNUM_INPUT_POS:%d\n", ni.num_input_pos);
    }
    fprintf(fp, "NASM_NINSTS_END\nASPEN_NASM_END\n");
    fclose(fp);
}

namespace {
struct NasmReader {
    FILE *fp;
    char buf[MAX_STRING_LEN];
    unsigned int line_no = 0;
    const char *expect(const char *tag) {
        if (!fgets(buf, sizeof buf, fp)) { ASPEN_ERR("ASPEN NASM file parse error: Unexpected EOF.\n"); return nullptr; }
        line_no++;
        buf[strcspn(buf, "\n")] = 0;
        char *p = buf;
        while (*p == ' ' || *p == '\t') p++;
        size_t n = strlen(tag);
        if (strncmp(p, tag, n) != 0) {
            ASPEN_ERR("Wrong ASPEN NASM file format at line %u, expected \"%s\", got \"%s\"\n", line_no, tag, p);
            return nullptr;
        }
        return p + n;
    }
    bool pair(long *a, long *b) {
        if (!fgets(buf, sizeof buf, fp)) return false;
        line_no++;
        return sscanf(buf, " %ld %ld", a, b) == 2;
    }
};
}  // namespace

extern "C" nasm_t *apu_load_nasm_from_file(char *filename, aspen_dnn_t *dnn) {
    if (!dnn) { ASPEN_ERR("ASPEN DNN NASM load error: dnn is null.\n"); return nullptr; }
    if (!filename) { ASPEN_ERR("ASPEN DNN NASM load error: filename is null.\n"); return nullptr; }
    FILE *fp = fopen(filename, "rb");
    if (!fp) { ASPEN_ERR("ASPEN DNN NASM load error: file %s not found.\n", filename); return nullptr; }
    NasmReader rd{fp};
    nasm_t *nasm = nullptr;
    const char *p;
    bool ok = false;
    unsigned int batch = 0, min_ninst = 0, flop = 0, seq = 0;
    unsigned long total_flops = 0;
    if (!rd.expect("ASPEN_NASM") || !rd.expect("DNN_NAME:")) goto done;
    if (!(p = rd.expect("NUM_BATCH:"))) goto done;
    batch = atoi(p);
    if (!(p = rd.expect("MIN_NINST_PER_LDATA:"))) goto done;
    min_ninst = atoi(p);
    if (!(p = rd.expect("TOTAL_FLOPS:"))) goto done;
    total_flops = atol(p);
    if (!(p = rd.expect("FLOP_PER_NINST:"))) goto done;
    flop = atoi(p);
    if (!(p = rd.expect("SEQ_LEN:"))) goto done;
    seq = atoi(p);
    // The file holds no geometry: tiles are regenerated from the header with the reference quanta.
    {
        TileQuanta saved = g_quanta;
        g_quanta = TileQuanta();
        nasm = nasm_create_tiles(dnn, flop, batch, min_ninst, seq);
        g_quanta = saved;
    }
    if (!nasm) goto done;
    nasm->total_flops = total_flops;
    if (!rd.expect("NASM_NINSTS:")) goto done;
    for (auto &ni : nasm->ninst) {
        long a, b;
        if (!(p = rd.expect("NINST_IDX:"))) goto done;
        if ((unsigned int)atoi(p) != ni.ninst_idx) { ASPEN_ERR("ASPEN NASM file %s parse error: NINST_IDX mismatch.\n", filename); goto done; }
        if (!rd.expect("NUM_CHILD_NINSTS:")) goto done;
        if (!(p = rd.expect("NUM_PARENT_NINSTS:"))) goto done;
        ni.parent_ninst_idx.assign((size_t)atoi(p), 0);
        if (!rd.expect("PARENT_NINSTS:")) goto done;
        for (size_t k = 0; k < ni.parent_ninst_idx.size(); k++) {
            if (!rd.pair(&a, &b) || a < 0 || (size_t)a >= ni.parent_ninst_idx.size() || b < 0 || b >= (long)nasm->num_ninst) goto done;
            ni.parent_ninst_idx[a] = (unsigned int)b;
        }
        if (!rd.expect("PARENT_NINSTS_END")) goto done;
        if (!(p = rd.expect("NUM_CHILD_NINSTS:"))) goto done;
        ni.child_ninst_idx.assign((size_t)atoi(p), 0);
        if (!rd.expect("CHILD_NINST_IDXES:")) goto done;
        for (size_t k = 0; k < ni.child_ninst_idx.size(); k++) {
            if (!rd.pair(&a, &b) || a < 0 || (size_t)a >= ni.child_ninst_idx.size() || b < 0 || b >= (long)nasm->num_ninst) goto done;
            ni.child_ninst_idx[a] = (unsigned int)b;
        }
        if (!rd.expect("CHILD_NINST_IDXES_END")) goto done;
        if (!(p = rd.expect("NUM_INPUT_POS:"))) goto done;
        ni.num_input_pos = atoi(p);
    }
    if (!rd.expect("NASM_NINSTS_END") || !rd.expect("ASPEN_NASM_END")) goto done;
    ok = true;
done:
    fclose(fp);
    if (!ok) {
        ASPEN_ERR("ASPEN NASM file %s parse error near line %u.\n", filename, rd.line_no);
        if (nasm) apu_destroy_nasm(nasm);
        return nullptr;
    }
    // A file only carries the reference's lists; recompute the true-dependency supplement.
    {
        ParentFinder pf(nasm);
        std::vector<unsigned int> scratch;
        for (auto &ni : nasm->ninst) { scratch.clear(); ni.extra_parent_idx.clear(); pf.run(ni, scratch, ni.extra_parent_idx); }
    }
    nasm->has_graph = true;
    return nasm;
}

// ---- read-only views ------------------------------------------------------------------------
extern "C" unsigned int aspen_b200_nasm_num_ldata(nasm_t *n) { return n ? n->num_ldata : 0; }
extern "C" unsigned int aspen_b200_nasm_num_ninst(nasm_t *n) { return n ? n->num_ninst : 0; }
extern "C" uint64_t aspen_b200_nasm_total_flops(nasm_t *n) { return n ? n->true_flops : 0; }
extern "C" void aspen_b200_nasm_ldata_info(nasm_t *n, unsigned int idx, unsigned int *out) {
    if (!n || idx >= n->num_ldata || !out) return;
    const nasm_ldata_t &l = n->ldata[idx];
    out[0] = l.layer->type; out[1] = l.layer->activation;
    out[2] = l.out_mat_dims[OUT_H]; out[3] = l.out_mat_dims[OUT_W]; out[4] = l.out_mat_stride;
    out[5] = l.ninst_tile_dims[OUT_H]; out[6] = l.ninst_tile_dims[OUT_W]; out[7] = l.num_ninst;
    out[8] = l.flop_per_output; out[9] = l.parent_ldata_idx_arr[PARENT_0]; out[10] = l.parent_ldata_idx_arr[PARENT_1];
    out[11] = (unsigned int)l.out_mat_mem_size;
}
extern "C" void aspen_b200_nasm_ninst_info(nasm_t *n, unsigned int idx, unsigned int *out) {
    if (!n || idx >= n->num_ninst || !out) return;
    const ninst_t &t = n->ninst[idx];
    out[0] = t.out_mat_pos[OUT_H]; out[1] = t.out_mat_pos[OUT_W]; out[2] = t.tile_dims[OUT_H]; out[3] = t.tile_dims[OUT_W];
    out[4] = (unsigned int)t.parent_ninst_idx.size(); out[5] = (unsigned int)t.child_ninst_idx.size(); out[6] = t.num_input_pos;
}
static unsigned int copy_list(const std::vector<unsigned int> &v, unsigned int *out, unsigned int cap) {
    for (unsigned int i = 0; i < v.size() && i < cap && out; i++) out[i] = v[i];
    return (unsigned int)v.size();
}
extern "C" unsigned int aspen_b200_nasm_ninst_parents(nasm_t *n, unsigned int idx, unsigned int *out, unsigned int cap) {
    return (!n || idx >= n->num_ninst) ? 0 : copy_list(n->ninst[idx].parent_ninst_idx, out, cap);
}
extern "C" unsigned int aspen_b200_nasm_ninst_children(nasm_t *n, unsigned int idx, unsigned int *out, unsigned int cap) {
    return (!n || idx >= n->num_ninst) ? 0 : copy_list(n->ninst[idx].child_ninst_idx, out, cap);
}
