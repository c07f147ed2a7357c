// Tiler: partitions every layer's output matrix (H = channels/features, W = pixels/tokens,
// column-major with padded column stride) into ninst tiles.
//
// The arithmetic must agree with the reference tiler exactly -- its .nasm loader re-runs the tiler
// and checks tile indices (ref src/apu_file_io.c:938-973), and tile ids are the graph's node ids.
// Sources followed: get_out_mat_info (src/apu_nasm.c:950-1023), get_ninst_tile_dims (1025-1060),
// init_nasm_ldata (1062-1182), init_ninst (468-478), position maps (1214-1327).
// The two quanta (64 rows / 12 columns in the reference, include/aspen.h:30-31) and the flop
// target are parameters here so a tensor-core-shaped profile can be produced by the same rules.
#include "internal.h"

TileQuanta g_quanta;

extern "C" void aspen_b200_set_tile_quanta(unsigned int h_min, unsigned int w_min, unsigned int flop_per_ninst) {
    g_quanta.h_min = h_min ? h_min : NINST_H_MIN;
    g_quanta.w_min = w_min ? w_min : NINST_W_MIN;
    g_quanta.flop_per_ninst = flop_per_ninst ? flop_per_ninst : 100000000u;
}
extern "C" void aspen_b200_set_tile_profile(int profile) {
    if (profile == 1) aspen_b200_set_tile_quanta(128, 128, 100000000u);
    else aspen_b200_set_tile_quanta(NINST_H_MIN, NINST_W_MIN, 100000000u);
}

static bool out_mat_info(nasm_ldata_t *ld) {
    const aspen_layer_t *l = ld->layer;
    const unsigned int *p = l->params;
    const unsigned int batch = ld->nasm->batch_size, seq = ld->nasm->tr_seq_len;
    unsigned int *dim = ld->out_mat_dims;
    switch (l->type) {
        case CONV_LAYER:
            ld->flop_per_output = 2 * p[WEIGHT_H] * p[WEIGHT_W] * p[IN_C];
            dim[OUT_H] = p[OUT_C]; dim[OUT_W] = p[OUT_H] * p[OUT_W] * batch;
            return true;
        case FC_LAYER:
            ld->flop_per_output = 2 * p[IN_C] * p[IN_H] * p[IN_W];
            dim[OUT_H] = p[OUT_C]; dim[OUT_W] = batch;
            return true;
        case MAXPOOL_LAYER: case AVGPOOL_LAYER:
            ld->flop_per_output = p[WEIGHT_H] * p[WEIGHT_W];
            dim[OUT_H] = p[OUT_C]; dim[OUT_W] = p[OUT_H] * p[OUT_W] * batch;
            return true;
        case INPUT_LAYER: case RESIDUAL_LAYER: case YOLO_LAYER: case APPEND_LAYER:
            ld->flop_per_output = 1;
            dim[OUT_H] = p[OUT_C]; dim[OUT_W] = p[OUT_H] * p[OUT_W] * batch;
            if (seq != 0) { dim[OUT_H] = p[MAT_M]; dim[OUT_W] = seq * batch; }
            return true;
        case SOFTMAX_LAYER:
            ld->flop_per_output = 1;
            dim[OUT_H] = p[OUT_C]; dim[OUT_W] = batch;
            return true;
        case MATMUL_LAYER:
            ld->flop_per_output = 2 * p[MAT_K];
            dim[OUT_H] = p[MAT_M]; dim[OUT_W] = seq * batch;
            return true;
        case K_ATTENTION_LAYER:
            ld->flop_per_output = p[NUM_HEAD] ? 2 * p[NUM_HIDDEN] / p[NUM_HEAD] : 0;
            dim[OUT_H] = seq; dim[OUT_W] = seq * p[NUM_HEAD] * batch;
            return true;
        case V_ATTENTION_LAYER:
            ld->flop_per_output = 2 * seq;
            dim[OUT_H] = p[MAT_M]; dim[OUT_W] = seq * batch;
            return true;
        case LAYERNORM_LAYER:
            ld->flop_per_output = 1;
            dim[OUT_H] = p[MAT_M]; dim[OUT_W] = seq * batch;
            return true;
        default:
            ASPEN_ERR("ERROR) Unsupported layer type %s\n", layer_type_str[l->type]);
            return false;
    }
}

// First guess: grow a (h_min x w_min) tile until it holds flop_per_ninst of work, rows first.
// Column quantum of a layer: the global one, except for convolutions staged by strided TMA boxes when tiles are
// whole MMA blocks -- their tiles are made of blocks of whole output rows (conv_block_width).
static unsigned int layer_w_quantum(const nasm_ldata_t *ld) {
    const TileQuanta &q = ld->nasm->quanta;
    if (q.w_min == 128 && conv_uses_row_blocks(ld->layer)) return conv_block_width(ld->layer->params[OUT_W], ld->layer->params[OUT_H]);
    return q.w_min;
}

static void initial_tile_dims(nasm_ldata_t *ld) {
    const TileQuanta &q = ld->nasm->quanta;
    const unsigned int w_min = layer_w_quantum(ld);
    unsigned int *t = ld->ninst_tile_dims;
    const unsigned int *dim = ld->out_mat_dims;
    t[OUT_H] = q.h_min < dim[OUT_H] ? q.h_min : dim[OUT_H];
    t[OUT_W] = w_min < dim[OUT_W] ? w_min : dim[OUT_W];
    if (t[OUT_H] == 0) t[OUT_H] = 1;
    if (t[OUT_W] == 0) t[OUT_W] = 1;
    const unsigned int want = ld->flop_per_output ? ld->nasm->flop_per_ninst / ld->flop_per_output : 0;
    while (t[OUT_H] * t[OUT_W] < want) {
        if (t[OUT_H] < dim[OUT_H]) t[OUT_H]++;
        else if (t[OUT_W] < dim[OUT_W]) t[OUT_W]++;
        else break;
    }
    t[OUT_H] = (unsigned int)round_up(t[OUT_H], q.h_min);
    if (ld->layer->type != FC_LAYER && ld->layer->type != SOFTMAX_LAYER)
        t[OUT_W] = (unsigned int)round_up(t[OUT_W], w_min);
}

void tiler_init_ldata(nasm_t *nasm, nasm_ldata_t *ld, aspen_layer_t *layer) {
    const TileQuanta &q = nasm->quanta;
    ld->nasm = nasm;
    ld->layer = layer;
    for (int i = 0; i < NUM_PARENT_ELEMENTS; i++) {
        ld->parent_ldata_idx_arr[i] = (unsigned int)-1;
        if (layer->parent_layers[i]) {
            unsigned int pidx = layer->parent_layers[i]->layer_idx;
            ld->parent_ldata_idx_arr[i] = pidx;
            nasm->ldata[pidx].num_child_ldata++;
        }
    }
    ld->flop_per_output = 1;
    out_mat_info(ld);
    initial_tile_dims(ld);
    unsigned int *t = ld->ninst_tile_dims;
    const unsigned int *dim = ld->out_mat_dims;
    const LAYER_TYPE type = layer->type;
    unsigned int unit_h = q.h_min, unit_w = layer_w_quantum(ld), hidden_per_head = 0;
    const bool whole_column = type == SOFTMAX_LAYER || type == APPEND_LAYER || type == YOLO_LAYER;
    if (whole_column) t[OUT_H] = (unsigned int)round_up(dim[OUT_H], q.h_min);
    if (type == SOFTMAX_LAYER) t[OUT_W] = 1;
    if (type == FC_LAYER && dim[OUT_W] < unit_w) unit_w = dim[OUT_W];
    // The reference cuts every layer that carries a head count into tiles of at most one head's rows and lets their
    // width shrink to 8 columns.  With tensor-core quanta the query / key / value projections (plain matmuls whose
    // consumers address heads by offset) keep whole MMA blocks instead: a 64-row tile stages half the FLOP per byte
    // of a 256-row one.
    const bool ref_quanta = q.h_min == NINST_H_MIN && q.w_min == NINST_W_MIN;
    const bool per_head = layer->params[NUM_HEAD] > 0 && (ref_quanta || type != MATMUL_LAYER);
    if (layer->params[NUM_HEAD] > 0) hidden_per_head = layer->params[NUM_HIDDEN] / layer->params[NUM_HEAD];
    if (per_head) {
        unit_w = 8;
        unit_h = hidden_per_head / 4;
    }
    unsigned int out_w = (unsigned int)round_up(dim[OUT_W], t[OUT_W]);
    unsigned int out_h = (unsigned int)round_up(dim[OUT_H], t[OUT_H]);
    const bool h_fixed = type == APPEND_LAYER || type == YOLO_LAYER;
    if (type != SOFTMAX_LAYER) {
        // Halve columns, then rows, until the layer has at least min_ninst_per_ldata tiles.
        while ((out_w / t[OUT_W]) * (out_h / t[OUT_H]) < nasm->min_ninst_per_ldata) {
            if (t[OUT_W] > unit_w) {
                t[OUT_W] /= 2;
                while (t[OUT_W] % unit_w != 0) t[OUT_W]++;
            } else if (t[OUT_H] > unit_h) {
                if (!h_fixed) {
                    t[OUT_H] /= 2;
                    while (t[OUT_H] % unit_h != 0) t[OUT_H]++;
                }
            }
            out_w = (unsigned int)round_up(dim[OUT_W], t[OUT_W]);
            out_h = (unsigned int)round_up(dim[OUT_H], t[OUT_H]);
            if (t[OUT_W] == unit_w && (t[OUT_H] == unit_h || h_fixed)) break;
            if (t[OUT_W] <= unit_w && (t[OUT_H] <= unit_h || h_fixed)) break;   // cannot shrink further
        }
    }
    if (per_head || type == LAYERNORM_LAYER) {
        // Transformer layers: a tile never straddles heads; layernorm and attention scores take a
        // whole column; the column count is rescaled to keep the tile area and made to divide seq.
        const unsigned int old_h = t[OUT_H];
        if (t[OUT_H] > hidden_per_head) t[OUT_H] = hidden_per_head;
        if (type == LAYERNORM_LAYER) t[OUT_H] = layer->params[MAT_M];
        else if (type == K_ATTENTION_LAYER) t[OUT_H] = (unsigned int)round_up(nasm->tr_seq_len, 8);
        else if (type == V_ATTENTION_LAYER) {
            if (hidden_per_head < t[OUT_H]) t[OUT_H] = hidden_per_head;
            while (hidden_per_head % t[OUT_H] != 0) t[OUT_H]++;
        }
        t[OUT_W] = (unsigned int)((float)t[OUT_W] * old_h / t[OUT_H]);
        if (t[OUT_W] > nasm->tr_seq_len) t[OUT_W] = nasm->tr_seq_len;
        if (t[OUT_W] == 0) t[OUT_W] = 1;
        while (nasm->tr_seq_len % t[OUT_W] != 0 && type != LAYERNORM_LAYER) t[OUT_W]++;
        out_w = (unsigned int)round_up(dim[OUT_W], t[OUT_W]);
        out_h = (unsigned int)round_up(dim[OUT_H], t[OUT_H]);
    }
    ld->out_mat_stride = out_h;
    ld->out_mat_mem_size = round_up((size_t)ld->out_mat_stride * out_w * layer->dnn->element_size, MEM_ALIGN);
    ld->num_ninst = (out_h / t[OUT_H]) * (out_w / t[OUT_W]);
}

// Tiles are numbered column-block major: idx = (w / tile_w) * tiles_per_column + h / tile_h.
void tiler_init_ninst(nasm_ldata_t *ld, ninst_t *ni, unsigned int ninst_idx) {
    ni->ldata = ld;
    ni->state = NINST_NOT_READY;
    ni->ninst_idx = ninst_idx;
    const unsigned int th = ld->ninst_tile_dims[OUT_H], tw = ld->ninst_tile_dims[OUT_W];
    const unsigned int per_col = (unsigned int)round_up(ld->out_mat_dims[OUT_H], th) / th;
    const unsigned int local = ninst_idx - ld->ninst_start;
    ni->out_mat_pos[OUT_H] = (local % per_col) * th;
    ni->out_mat_pos[OUT_W] = (local / per_col) * tw;
    ni->tile_dims[OUT_W] = ni->out_mat_pos[OUT_W] + tw > ld->out_mat_dims[OUT_W] ? ld->out_mat_dims[OUT_W] - ni->out_mat_pos[OUT_W] : tw;
    ni->tile_dims[OUT_H] = ni->out_mat_pos[OUT_H] + th > ld->out_mat_dims[OUT_H] ? ld->out_mat_dims[OUT_H] - ni->out_mat_pos[OUT_H] : th;
    const aspen_layer_t *l = ld->layer;
    if (l->type == CONV_LAYER || l->type == MAXPOOL_LAYER || l->type == AVGPOOL_LAYER)   // ref src/apu_nasm.c:37-46
        ni->num_input_pos = ni->tile_dims[OUT_W] * l->params[WEIGHT_H] * l->params[WEIGHT_W];
}

static bool image_like(const aspen_layer_t *l) {
    switch (l->type) {
        case CONV_LAYER: case MAXPOOL_LAYER: case AVGPOOL_LAYER: case INPUT_LAYER: case RESIDUAL_LAYER:
        case YOLO_LAYER: case APPEND_LAYER: return true;
        default: return false;
    }
}

void out_mat_pos_from_tensor_pos(const nasm_ldata_t *ld, const unsigned int *tp, unsigned int *mp) {
    const aspen_layer_t *l = ld->layer;
    const unsigned int *p = l->params;
    const unsigned int seq = ld->nasm->tr_seq_len;
    if (image_like(l)) {
        if (p[MAT_M] == 0) {
            mp[OUT_H] = tp[OUT_C];
            mp[OUT_W] = tp[BATCH] * p[OUT_H] * p[OUT_W] + tp[OUT_H] * p[OUT_W] + tp[OUT_W];
        } else {
            mp[OUT_H] = tp[MAT_M];
            mp[OUT_W] = tp[BATCH] * seq + tp[MAT_N];
        }
    } else if (l->type == FC_LAYER || l->type == SOFTMAX_LAYER) {
        mp[OUT_H] = tp[OUT_C];
        mp[OUT_W] = tp[BATCH];
    } else if (l->type == K_ATTENTION_LAYER) {
        mp[OUT_H] = tp[MAT_M];
        mp[OUT_W] = tp[BATCH] * seq * p[NUM_HEAD] + tp[NUM_HEAD] * seq + tp[MAT_N];
    } else {   // matmul, layernorm, attention_v
        mp[OUT_H] = tp[MAT_M];
        mp[OUT_W] = tp[BATCH] * seq + tp[MAT_N];
    }
}

void tensor_pos_from_out_mat_pos(const nasm_ldata_t *ld, const unsigned int *mp, unsigned int *tp) {
    const aspen_layer_t *l = ld->layer;
    const unsigned int *p = l->params;
    const unsigned int seq = ld->nasm->tr_seq_len;
    if (image_like(l)) {
        if (p[MAT_M] == 0) {
            const unsigned int hw = p[OUT_H] * p[OUT_W];
            tp[BATCH] = mp[OUT_W] / hw;
            tp[OUT_C] = mp[OUT_H];
            tp[OUT_H] = (mp[OUT_W] % hw) / p[OUT_W];
            tp[OUT_W] = mp[OUT_W] % p[OUT_W];
        } else {
            tp[BATCH] = mp[OUT_W] / seq;
            tp[MAT_N] = mp[OUT_W] % seq;
            tp[MAT_M] = mp[OUT_H];
            tp[OUT_C] = tp[MAT_M];
            tp[OUT_H] = 1;
            tp[OUT_W] = tp[MAT_N];
        }
    } else if (l->type == FC_LAYER || l->type == SOFTMAX_LAYER) {
        tp[BATCH] = mp[OUT_W];
        tp[OUT_C] = mp[OUT_H];
        tp[OUT_H] = 1;
        tp[OUT_W] = 1;
    } else if (l->type == K_ATTENTION_LAYER) {
        tp[BATCH] = mp[OUT_W] / (p[NUM_HEAD] * seq);
        tp[NUM_HEAD] = (mp[OUT_W] % (p[NUM_HEAD] * seq)) / seq;
        tp[MAT_N] = mp[OUT_W] % seq;
        tp[MAT_M] = mp[OUT_H];
    } else {
        tp[BATCH] = mp[OUT_W] / seq;
        tp[MAT_N] = mp[OUT_W] % seq;
        tp[MAT_M] = mp[OUT_H];
    }
}

static std::atomic<unsigned int> g_nasm_counter{0};

// ref src/apu_nasm.c:490-542
nasm_t *nasm_create_tiles(aspen_dnn_t *dnn, unsigned int flop_per_ninst, unsigned int batch, unsigned int min_ninst, unsigned int seq) {
    if (!dnn) { ASPEN_ERR("nasm creation: dnn is NULL\n"); return nullptr; }
    if (min_ninst < 1) { ASPEN_ERR("ERROR: min_ninst_per_ldata should be at least 1\n"); return nullptr; }
    nasm_t *nasm = new nasm_t();
    nasm->dnn = dnn;
    nasm->tr_seq_len = seq;
    nasm->flop_per_ninst = flop_per_ninst > 0 ? flop_per_ninst : 1;
    nasm->batch_size = batch > 0 ? batch : 1;
    nasm->nasm_id = g_nasm_counter.fetch_add(1);
    nasm->min_ninst_per_ldata = min_ninst;
    nasm->quanta = g_quanta;
    nasm->quanta.flop_per_ninst = nasm->flop_per_ninst;
    nasm->num_ldata = dnn->num_layers;
    nasm->ldata.resize(nasm->num_ldata);
    for (unsigned int i = 0; i < nasm->num_ldata; i++) tiler_init_ldata(nasm, &nasm->ldata[i], &dnn->layers[i]);
    unsigned int total = 0;
    for (auto &ld : nasm->ldata) { ld.ninst_start = total; total += ld.num_ninst; }
    nasm->num_ninst = total;
    nasm->ninst.resize(total);
    for (auto &ld : nasm->ldata)
        for (unsigned int j = 0; j < ld.num_ninst; j++) tiler_init_ninst(&ld, &nasm->ninst[ld.ninst_start + j], ld.ninst_start + j);
    for (unsigned int i = 0; i < nasm->num_ldata; i++) {   // child layer lists, duplicates kept
        for (unsigned int c = 0; c < nasm->num_ldata; c++)
            for (int k = 0; k < NUM_PARENT_ELEMENTS; k++)
                if (nasm->ldata[c].parent_ldata_idx_arr[k] == i) nasm->ldata[i].child_ldata_idx.push_back(c);
    }
    // total_flops is what the .nasm header carries: the reference sums 32-bit per-layer products
    // (src/apu_nasm.c:704-711), which wrap for large layers (its shipped vgg16_B3.nasm shows it);
    // true_flops is the unwrapped count the benchmark reports.
    nasm->total_flops = 0;
    nasm->true_flops = 0;
    for (auto &ld : nasm->ldata) {
        nasm->total_flops += (unsigned int)(ld.flop_per_output * ld.out_mat_dims[OUT_H] * ld.out_mat_dims[OUT_W]);
        nasm->true_flops += (uint64_t)ld.flop_per_output * ld.out_mat_dims[OUT_H] * ld.out_mat_dims[OUT_W];
    }
    dnn->ref_nasms.fetch_add(1);
    return nasm;
}
