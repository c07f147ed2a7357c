// aspen_dnn_t: tensors, weight files (ASPEN_DATA .bin, .aspen), create/destroy.
#include "internal.h"

#include <cmath>

// ---- error channel -----------------------------------------------------------------------
static thread_local char g_last_error[1024] = "";

void aspen_error(const char *file, int line, const char *fmt, ...) {
    char msg[900];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof msg, fmt, ap);
    va_end(ap);
    snprintf(g_last_error, sizeof g_last_error, "(%s:%d)%s", file, line, msg);
    fprintf(stderr, "\033[0;31m%s\033[0m", g_last_error);
}
extern "C" const char *aspen_b200_last_error(void) { return g_last_error; }

// ---- name tables (ref: src/util.c:3-41) ---------------------------------------------------
extern "C" {
char *ninst_state_str[NUM_NINST_STATES] = {(char *)"NINST_NOT_READY", (char *)"NINST_READY", (char *)"NINST_COMPLETED"};
char *layer_type_str[NUM_LAYER_ELEMENTS] = {
    (char *)"NO_LAYER_TYPE", (char *)"INPUT_LAYER", (char *)"CONV_LAYER", (char *)"FC_LAYER", (char *)"RESIDUAL_LAYER",
    (char *)"BATCHNORM_LAYER", (char *)"YOLO_LAYER", (char *)"APPEND_LAYER", (char *)"ACTIVATION_LAYER",
    (char *)"MAXPOOL_LAYER", (char *)"AVGPOOL_LAYER", (char *)"ROUTE_LAYER", (char *)"SOFTMAX_LAYER",
    (char *)"MATMUL_LAYER", (char *)"LAYERNORM_LAYER", (char *)"K_ATTENTION_LAYER", (char *)"V_ATTENTION_LAYER"};
char *param_type_str[NUM_PARAM_ELEMENTS] = {
    (char *)"OUT_W", (char *)"OUT_H", (char *)"OUT_C", (char *)"BATCH", (char *)"IN_W", (char *)"IN_H", (char *)"IN_C",
    (char *)"WEIGHT_W", (char *)"WEIGHT_H", (char *)"SUB_C", (char *)"STRIDE", (char *)"PADDING", (char *)"DILATION",
    (char *)"GROUPS", (char *)"NUM_HIDDEN", (char *)"NUM_HEAD", (char *)"NUM_SEQ", (char *)"MAT_M", (char *)"MAT_N",
    (char *)"MAT_K", (char *)"SUB_M", (char *)"MASKED", (char *)"FORM_BYTES"};
char *tensor_type_str[NUM_TENSORS] = {
    (char *)"NULL_TENSOR", (char *)"OUTPUT_TENSOR", (char *)"INPUT_TENSOR", (char *)"WEIGHT_TENSOR", (char *)"BIAS_TENSOR",
    (char *)"COL_IDX_TENSOR", (char *)"ANCHOR_TENSOR", (char *)"BN_VAR_TENSOR", (char *)"BN_MEAN_TENSOR",
    (char *)"BN_WEIGHT_TENSOR"};
char *parent_type_str[NUM_PARENT_ELEMENTS] = {(char *)"PARENT_NONE", (char *)"PARENT_0", (char *)"PARENT_1", (char *)"PARENT_WEIGHT"};
char *activation_type_str[NUM_ACTIVATIONS] = {
    (char *)"NO_ACTIVATION", (char *)"SIGMOID", (char *)"LINEAR", (char *)"TANH", (char *)"RELU", (char *)"LEAKY_RELU",
    (char *)"ELU", (char *)"SELU", (char *)"GELU", (char *)"GELU_ACCURATE"};
char *rpool_cond_str[NUM_RPOOL_CONDS] = {(char *)"RPOOL_DNN", (char *)"RPOOL_LAYER_TYPE", (char *)"RPOOL_LAYER_IDX",
                                         (char *)"RPOOL_NASM", (char *)"RPOOL_DSE"};
}

// ---- tensors -----------------------------------------------------------------------------
aspen_tensor_t *tensor_create(const unsigned int *params, const LAYER_PARAMS *order, int num_dims, unsigned int elem) {
    aspen_tensor_t *t = new aspen_tensor_t();
    t->num_dims = num_dims;
    t->element_size = elem;
    t->num_elements = 1;
    for (int i = 0; i < num_dims; i++) {
        t->data_dim_order[i] = order[i];
        t->dims[order[i]] = params[order[i]];
        t->num_elements *= params[order[i]];
    }
    return t;
}

static void tensor_alloc(aspen_tensor_t *t) {
    free(t->data);
    t->data = calloc((size_t)t->num_elements + 8, t->element_size);
}

void tensor_destroy(aspen_tensor_t *t) {
    if (!t) return;
    free(t->data);
    delete t;
}

unsigned int tensor_idx_from_pos(const aspen_tensor_t *t, const unsigned int *pos) {
    unsigned int idx = 0;
    for (unsigned int i = 0; i < t->num_dims; i++) {
        LAYER_PARAMS d = t->data_dim_order[i];
        idx = idx * t->dims[d] + pos[d];
    }
    return idx;
}

void tensor_pos_from_idx(const aspen_tensor_t *t, unsigned int idx, unsigned int *pos) {
    for (int i = (int)t->num_dims - 1; i >= 0; i--) {
        LAYER_PARAMS d = t->data_dim_order[i];
        pos[d] = idx % t->dims[d];
        idx /= t->dims[d];
    }
}

unsigned int layer_contraction_k(const aspen_layer_t *l) {
    const unsigned int *p = l->params;
    switch (l->type) {
        case CONV_LAYER: return p[WEIGHT_H] * p[WEIGHT_W] * p[IN_C];
        case FC_LAYER: return p[IN_C] * p[IN_H] * p[IN_W];
        case MATMUL_LAYER: return p[MAT_K];
        default: return 0;
    }
}

unsigned int layer_weight_rows(const aspen_layer_t *l) {
    switch (l->type) {
        case CONV_LAYER: case FC_LAYER: return l->params[OUT_C];
        case MATMUL_LAYER: case LAYERNORM_LAYER: return l->params[MAT_M];
        default: return 0;
    }
}

// Canonical dim orders of the host weight tensors (rows first, then the contraction in the order
// the tile kernels walk it: ref src/tiled_kernels.c:21-36 for conv, 502-516 for connected).
static int weight_order(const aspen_layer_t *l, LAYER_PARAMS *order) {
    switch (l->type) {
        case CONV_LAYER: order[0] = OUT_C; order[1] = WEIGHT_H; order[2] = WEIGHT_W; order[3] = IN_C; return 4;
        case FC_LAYER: order[0] = OUT_C; order[1] = IN_H; order[2] = IN_W; order[3] = IN_C; return 4;
        case MATMUL_LAYER: order[0] = MAT_M; order[1] = MAT_K; return 2;
        case LAYERNORM_LAYER: order[0] = MAT_M; return 1;
        default: return 0;
    }
}
// Dim order of the same tensor inside an ASPEN_DATA weight file (ref src/apu_file_io.c:226-255).
static int file_weight_order(const aspen_layer_t *l, LAYER_PARAMS *order) {
    switch (l->type) {
        case CONV_LAYER: order[0] = OUT_C; order[1] = IN_C; order[2] = WEIGHT_H; order[3] = WEIGHT_W; return 4;
        case FC_LAYER: order[0] = OUT_C; order[1] = IN_C; order[2] = IN_H; order[3] = IN_W; return 4;
        case MATMUL_LAYER: order[0] = MAT_M; order[1] = MAT_K; return 2;
        case LAYERNORM_LAYER: order[0] = MAT_M; return 1;
        default: return 0;
    }
}

// Copy src (packed in src_order) into dst (packed in dst's own order); same dims.
static void tensor_permute_from(aspen_tensor_t *dst, const float *src, const LAYER_PARAMS *src_order, int nd) {
    aspen_tensor_t view = *dst;
    for (int i = 0; i < nd; i++) view.data_dim_order[i] = src_order[i];
    unsigned int pos[NUM_PARAM_ELEMENTS] = {};
    float *out = (float *)dst->data;
    for (unsigned int i = 0; i < dst->num_elements; i++) {
        tensor_pos_from_idx(&view, i, pos);
        out[tensor_idx_from_pos(dst, pos)] = src[i];
    }
}

// rand()-driven +-0.3 fill in the element order the reference uses (ref src/apu.c:345-354,418-421),
// so a dnn created without a weight file holds the same numbers under the same rand() state.
static void fill_random(float *buf, unsigned int n) {
    for (unsigned int i = 0; i < n; i++) buf[i] = (((float)rand() / (float)RAND_MAX) - 0.5) * 2 * 0.3f;
}

static void create_layer_tensors(aspen_layer_t *l) {
    LAYER_PARAMS order[MAX_TENSOR_DIMS];
    int nd = weight_order(l, order);
    if (nd == 0) return;
    l->tensors[WEIGHT_TENSOR] = tensor_create(l->params, order, nd, l->dnn->element_size);
    tensor_alloc(l->tensors[WEIGHT_TENSOR]);
    LAYER_PARAMS border[1] = {order[0]};
    l->tensors[BIAS_TENSOR] = tensor_create(l->params, border, 1, l->dnn->element_size);
    tensor_alloc(l->tensors[BIAS_TENSOR]);
    aspen_tensor_t *w = l->tensors[WEIGHT_TENSOR];
    std::vector<float> tmp(w->num_elements);
    fill_random(tmp.data(), w->num_elements);
    if (l->type == FC_LAYER) {   // the reference draws connected weights in (o, c, h, w) order
        LAYER_PARAMS draw[4] = {OUT_C, IN_C, IN_H, IN_W};
        tensor_permute_from(w, tmp.data(), draw, 4);
    } else {
        memcpy(w->data, tmp.data(), sizeof(float) * w->num_elements);
    }
    fill_random((float *)l->tensors[BIAS_TENSOR]->data, l->tensors[BIAS_TENSOR]->num_elements);
}

// ---- ASPEN_DATA weight file ----------------------------------------------------------------
namespace {
struct LineReader {
    FILE *fp;
    unsigned int line_no = 0;
    char buf[MAX_STRING_LEN];
    // Reads one text line, skips leading blanks, requires `tag` as prefix; returns the remainder.
    const char *expect(const char *tag, bool quiet_eof = false) {
        if (!fgets(buf, sizeof buf, fp)) {
            if (!quiet_eof) ASPEN_ERR("ASPEN file parse error: Unexpected EOF.\n");
            return nullptr;
        }
        line_no++;
        buf[strcspn(buf, "\n")] = 0;
        char *p = buf;
        while (*p == ' ' || *p == '\t') p++;
        size_t n = strlen(tag);
        if (strncmp(p, tag, n) != 0) {
            ASPEN_ERR("Wrong ASPEN file format at line %u, expected \"%s\", got \"%s\"\n", line_no, tag, p);
            return nullptr;
        }
        return p + n;
    }
    bool pair(int *a, long *b) {
        if (!fgets(buf, sizeof buf, fp)) return false;
        line_no++;
        return sscanf(buf, " %d %ld", a, b) == 2;
    }
};

void fold_batchnorm(const float *var, const float *mean, const float *gamma, float *weight, float *bias,
                    unsigned int rows, unsigned int k) {   // ref src/util.c:259-276
    const double eps = 1e-5;
    for (unsigned int i = 0; i < rows; i++) {
        float inv = sqrtf(var[i] + eps);
        for (unsigned int j = 0; j < k; j++) weight[(size_t)i * k + j] = weight[(size_t)i * k + j] * gamma[i] / inv;
        bias[i] = bias[i] - gamma[i] * mean[i] / inv;
    }
}
}  // namespace

static bool load_weight_file(aspen_dnn_t *dnn, const char *path) {
    FILE *fp = fopen(path, "rb");
    if (!fp) {
        ASPEN_ERR("ASPEN DNN file %s not found.\n", path);
        return false;
    }
    LineReader rd{fp};
    bool ok = false;
    std::vector<float> bn_var, bn_mean, bn_gamma;
    const char *p;
    if (!rd.expect("ASPEN_DATA")) goto done;
    p = rd.expect("LAYER:");
    while (p) {
        int file_layer = atoi(p);
        aspen_layer_t *layer = nullptr;
        int seen = 0;
        for (auto &l : dnn->layers) {
            if (l.type == CONV_LAYER || l.type == FC_LAYER || l.type == MATMUL_LAYER || l.type == LAYERNORM_LAYER)
                if (++seen == file_layer) { layer = &l; break; }
        }
        if (!layer) { ASPEN_ERR("ASPEN DNN file %s parse error: Invalid file LAYER %d.\n", path, file_layer); goto done; }
        if (!(p = rd.expect("TENSOR_TYPE:"))) goto done;
        std::string kind = p;
        if (!(p = rd.expect("DATA_SIZE:"))) goto done;
        size_t bytes = (size_t)atol(p);
        if (!rd.expect("DATA_START:")) goto done;
        std::vector<float> data(bytes / sizeof(float) + 1);
        if (bytes && fread(data.data(), bytes, 1, fp) != 1) { ASPEN_ERR("ASPEN DNN file %s parse error: Failed to read data.\n", path); goto done; }
        if (!rd.expect("DATA_END")) goto done;
        if (kind == "WEIGHT") {
            aspen_tensor_t *w = layer->tensors[WEIGHT_TENSOR];
            if (!w || (size_t)w->num_elements * w->element_size != bytes) {
                ASPEN_ERR("ASPEN DNN file %s parse error: Layer %u WEIGHT_TENSOR size mismatch. Tensor: %zu, File: %zu.\n",
                          path, layer->layer_idx, w ? (size_t)w->num_elements * w->element_size : (size_t)0, bytes);
                goto done;
            }
            LAYER_PARAMS forder[MAX_TENSOR_DIMS];
            int nd = file_weight_order(layer, forder);
            tensor_permute_from(w, data.data(), forder, nd);
        } else if (kind == "BIAS") {
            aspen_tensor_t *b = layer->tensors[BIAS_TENSOR];
            if (!b || (size_t)b->num_elements * b->element_size != bytes) {
                ASPEN_ERR("ASPEN DNN file %s parse error: Layer %u BIAS_TENSOR size mismatch.\n", path, layer->layer_idx);
                goto done;
            }
            memcpy(b->data, data.data(), bytes);
        } else if (kind == "BN_VAR") { bn_var.assign(data.begin(), data.begin() + bytes / 4);
        } else if (kind == "BN_MEAN") { bn_mean.assign(data.begin(), data.begin() + bytes / 4);
        } else if (kind == "BN_WEIGHT") { bn_gamma.assign(data.begin(), data.begin() + bytes / 4);
        } else if (kind == "INPUT" || kind == "OUTPUT") {
            // carried by the format, unused by the runtime
        } else {
            ASPEN_ERR("ASPEN DNN file %s file layer %d parse error: Invalid TENSOR_TYPE %s.\n", path, file_layer, kind.c_str());
            goto done;
        }
        if (!bn_var.empty() && !bn_mean.empty() && !bn_gamma.empty()) {
            unsigned int rows = layer_weight_rows(layer), k = layer_contraction_k(layer);
            if (bn_var.size() >= rows && bn_mean.size() >= rows && bn_gamma.size() >= rows && layer->tensors[WEIGHT_TENSOR])
                fold_batchnorm(bn_var.data(), bn_mean.data(), bn_gamma.data(), (float *)layer->tensors[WEIGHT_TENSOR]->data,
                               (float *)layer->tensors[BIAS_TENSOR]->data, rows, k);
            bn_var.clear(); bn_mean.clear(); bn_gamma.clear();
        }
        if (!rd.expect("LAYER_END")) goto done;
        p = rd.expect("LAYER:", true);
    }
    ok = true;
done:
    fclose(fp);
    return ok;
}

// ---- public: create / destroy --------------------------------------------------------------
extern "C" aspen_dnn_t *apu_create_dnn(char *input_path, char *data_path) {
    if (!input_path) { ASPEN_ERR("apu_create_dnn: input_path is NULL\n"); return nullptr; }
    aspen_dnn_t *dnn = parse_cfg_file(input_path);
    if (!dnn) return nullptr;
    for (auto &l : dnn->layers) create_layer_tensors(&l);
    if (data_path) load_weight_file(dnn, data_path);
    return dnn;
}

static void free_dnn(aspen_dnn_t *dnn) {
    engine_release_dnn(dnn);
    for (auto &l : dnn->layers)
        for (auto &t : l.tensors) { tensor_destroy(t); t = nullptr; }
    delete dnn;
}

extern "C" void apu_destroy_dnn(aspen_dnn_t *dnn) {
    if (!dnn) return;
    if (dnn->ref_nasms.load() != 0) {
        ASPEN_ERR("Cannot destroy dnn %s with %d nasms still referencing it.\n", dnn->name, dnn->ref_nasms.load());
        return;
    }
    free_dnn(dnn);
}

// ---- .aspen codec ---------------------------------------------------------------------------
// The file stores conv / connected / matmul weights in the reference's AVX2 packing
// [rows/8][K][8] with an explicit SUB_C (SUB_M) inner dim (ref src/apu.c:14-40, saved verbatim by
// src/apu_file_io.c:434-501).  We write that layout and convert back on load, so files travel
// both ways between the two libraries.
static const unsigned int kPack = 8;

static void save_tensor(FILE *fp, const aspen_layer_t *l, int ti, const aspen_tensor_t *t) {
    aspen_tensor_t hdr = *t;
    std::vector<float> packed;
    const float *payload = (const float *)t->data;
    bool is_packed_weight = ti == WEIGHT_TENSOR && (l->type == CONV_LAYER || l->type == FC_LAYER || l->type == MATMUL_LAYER);
    if (is_packed_weight) {
        LAYER_PARAMS row_dim = t->data_dim_order[0];
        LAYER_PARAMS sub = l->type == MATMUL_LAYER ? SUB_M : SUB_C;
        unsigned int rows = t->dims[row_dim], k = t->num_elements / rows, groups = (rows + kPack - 1) / kPack;
        packed.assign((size_t)groups * k * kPack, 0.f);
        for (unsigned int r = 0; r < rows; r++)
            for (unsigned int j = 0; j < k; j++)
                packed[((size_t)(r / kPack) * k + j) * kPack + r % kPack] = payload[(size_t)r * k + j];
        hdr.dims[row_dim] = groups;
        hdr.dims[sub] = kPack;
        hdr.data_dim_order[hdr.num_dims++] = sub;
        hdr.num_elements = (unsigned int)packed.size();
        payload = packed.data();
    }
    fprintf(fp, "\t\t%d 1\n\t\tNUM_DIMS:%d\n\t\tDATA_DIM_ORDER:\n", ti, hdr.num_dims);
    for (int k = 0; k < MAX_TENSOR_DIMS; k++) fprintf(fp, "\t\t\t%d %d\n", k, hdr.data_dim_order[k]);
    fprintf(fp, "\t\tDATA_DIM_ORDER_END\n\t\tTENSOR_DIMS:\n");
    for (int k = 0; k < NUM_PARAM_ELEMENTS; k++) fprintf(fp, "\t\t\t%d %d\n", k, hdr.dims[k]);
    fprintf(fp, "\t\tTENSOR_DIMS_END\n\t\tTENSOR_DATA:\n");
    fwrite(payload, t->element_size, hdr.num_elements, fp);
    fprintf(fp, "\t\tTENSOR_DATA_END\n");
}

extern "C" void apu_save_dnn_to_file(aspen_dnn_t *dnn, char *filename) {
    if (!dnn || !filename) { ASPEN_ERR("apu_save_dnn_to_file: NULL argument\n"); return; }
    FILE *fp = fopen(filename, "wb");
    if (!fp) { ASPEN_ERR("Error: apu_save_dnn_to_file Failed to open file %s for writing\n", filename); return; }
    fprintf(fp, "ASPEN_DNN\nASPEN_BUILD:aspen_b200\nDNN_NAME:%s\nDNN_ELEMENT_SIZE:%d\nNUM_LAYERS:%d\n", dnn->name,
            dnn->element_size, dnn->num_layers);
    for (auto &l : dnn->layers) {
        fprintf(fp, "\tLAYER_IDX:%d\n\tLAYER_TYPE:%d\n\tLAYER_ACTIVATION:%d\n\tLAYER_PARENTS:\n", l.layer_idx, l.type, l.activation);
        for (int j = 0; j < NUM_PARENT_ELEMENTS; j++)
            fprintf(fp, "\t\t%d %d\n", j, l.parent_layers[j] ? (int)l.parent_layers[j]->layer_idx : -1);
        fprintf(fp, "\tLAYER_PARENTS_END\n\tLAYER_PARAMS:\n");
        for (int j = 0; j < NUM_PARAM_ELEMENTS; j++) fprintf(fp, "\t\t%d %d\n", j, l.params[j]);
        fprintf(fp, "\tLAYER_PARAMS_END\n\tLAYER_TENSORS:\n");
        for (int j = 0; j < NUM_TENSORS; j++) {
            if (l.tensors[j]) save_tensor(fp, &l, j, l.tensors[j]);
            else fprintf(fp, "\t\t%d -1\n", j);
        }
        fprintf(fp, "\tLAYER_TENSORS_END\n");
    }
    fprintf(fp, "ASPEN_DNN_END\n");
    fclose(fp);
}

extern "C" aspen_dnn_t *apu_load_dnn_from_file(char *filename) {
    if (!filename) { ASPEN_ERR("apu_load_dnn_from_file: filename is NULL\n"); return nullptr; }
    FILE *fp = fopen(filename, "rb");
    if (!fp) { ASPEN_ERR("ASPEN DNN file %s not found.\n", filename); return nullptr; }
    LineReader rd{fp};
    aspen_dnn_t *dnn = nullptr;
    const char *p;
    bool ok = false;
    char name[MAX_STRING_LEN] = {};
    if (!rd.expect("ASPEN_DNN") || !rd.expect("ASPEN_BUILD:")) goto done;
    if (!(p = rd.expect("DNN_NAME:"))) goto done;
    strncpy(name, p, MAX_STRING_LEN - 1);
    dnn = new aspen_dnn_t();
    strncpy(dnn->name, name, MAX_STRING_LEN - 1);
    if (!(p = rd.expect("DNN_ELEMENT_SIZE:"))) goto done;
    dnn->element_size = (unsigned int)atol(p);
    if (!(p = rd.expect("NUM_LAYERS:"))) goto done;
    dnn->num_layers = atoi(p);
    dnn->layers.resize(dnn->num_layers);
    for (unsigned int i = 0; i < dnn->num_layers; i++) {
        aspen_layer_t *l = &dnn->layers[i];
        l->dnn = dnn;
        int a; long b;
        if (!(p = rd.expect("LAYER_IDX:"))) goto done;
        l->layer_idx = atoi(p);
        if (!(p = rd.expect("LAYER_TYPE:"))) goto done;
        l->type = (LAYER_TYPE)atoi(p);
        if (!(p = rd.expect("LAYER_ACTIVATION:"))) goto done;
        l->activation = (LAYER_ACT)atoi(p);
        if (!rd.expect("LAYER_PARENTS:")) goto done;
        for (int j = 0; j < NUM_PARENT_ELEMENTS; j++) {
            if (!rd.pair(&a, &b) || a < 0 || a >= NUM_PARENT_ELEMENTS || b >= (long)dnn->num_layers) goto done;
            l->parent_layers[a] = b < 0 ? nullptr : &dnn->layers[b];
        }
        if (!rd.expect("LAYER_PARENTS_END") || !rd.expect("LAYER_PARAMS:")) goto done;
        for (int j = 0; j < NUM_PARAM_ELEMENTS; j++) {
            if (!rd.pair(&a, &b) || a < 0 || a >= NUM_PARAM_ELEMENTS) goto done;
            l->params[a] = (unsigned int)b;
        }
        if (!rd.expect("LAYER_PARAMS_END") || !rd.expect("LAYER_TENSORS:")) goto done;
        for (int j = 0; j < NUM_TENSORS; j++) {
            if (!rd.pair(&a, &b) || a < 0 || a >= NUM_TENSORS) goto done;
            if (b == -1) continue;
            aspen_tensor_t raw;
            raw.element_size = dnn->element_size;
            if (!(p = rd.expect("NUM_DIMS:"))) goto done;
            raw.num_dims = atoi(p);
            if (raw.num_dims > MAX_TENSOR_DIMS) goto done;
            if (!rd.expect("DATA_DIM_ORDER:")) goto done;
            for (int k = 0; k < MAX_TENSOR_DIMS; k++) {
                int di; long dv;
                if (!rd.pair(&di, &dv) || di < 0 || di >= MAX_TENSOR_DIMS || dv < 0 || dv >= NUM_PARAM_ELEMENTS) goto done;
                raw.data_dim_order[di] = (LAYER_PARAMS)dv;
            }
            if (!rd.expect("DATA_DIM_ORDER_END") || !rd.expect("TENSOR_DIMS:")) goto done;
            for (int k = 0; k < NUM_PARAM_ELEMENTS; k++) {
                int di; long dv;
                if (!rd.pair(&di, &dv) || di < 0 || di >= NUM_PARAM_ELEMENTS) goto done;
                raw.dims[di] = (unsigned int)dv;
            }
            if (!rd.expect("TENSOR_DIMS_END") || !rd.expect("TENSOR_DATA:")) goto done;
            raw.num_elements = 1;
            for (unsigned int k = 0; k < raw.num_dims; k++) raw.num_elements *= raw.dims[raw.data_dim_order[k]];
            std::vector<float> data((size_t)raw.num_elements + 1);
            if (raw.num_elements && fread(data.data(), dnn->element_size, raw.num_elements, fp) != raw.num_elements) goto done;
            if (!rd.expect("TENSOR_DATA_END")) goto done;
            LAYER_PARAMS last = raw.num_dims ? raw.data_dim_order[raw.num_dims - 1] : OUT_W;
            aspen_tensor_t *t;
            if (a == WEIGHT_TENSOR && (last == SUB_C || last == SUB_M) && raw.num_dims >= 2) {
                LAYER_PARAMS order[MAX_TENSOR_DIMS];
                int nd = weight_order(l, order);
                t = tensor_create(l->params, order, nd, dnn->element_size);
                tensor_alloc(t);
                unsigned int rows = t->dims[order[0]], k = t->num_elements / rows, sub = raw.dims[last];
                float *out = (float *)t->data;
                for (unsigned int r = 0; r < rows; r++)
                    for (unsigned int c = 0; c < k; c++)
                        out[(size_t)r * k + c] = data[((size_t)(r / sub) * k + c) * sub + r % sub];
            } else {
                t = new aspen_tensor_t(raw);
                t->data = nullptr;
                tensor_alloc(t);
                memcpy(t->data, data.data(), (size_t)raw.num_elements * dnn->element_size);
            }
            l->tensors[a] = t;
        }
        if (!rd.expect("LAYER_TENSORS_END")) goto done;
    }
    ok = rd.expect("ASPEN_DNN_END") != nullptr;
done:
    fclose(fp);
    if (!ok) {
        ASPEN_ERR("ASPEN DNN file %s parse error near line %u.\n", filename, rd.line_no);
        if (dnn) free_dnn(dnn);
        return nullptr;
    }
    return dnn;
}

// ---- read-only views ------------------------------------------------------------------------
extern "C" unsigned int aspen_b200_dnn_num_layers(aspen_dnn_t *dnn) { return dnn ? dnn->num_layers : 0; }
extern "C" void aspen_b200_dnn_layer_params(aspen_dnn_t *dnn, unsigned int idx, unsigned int *out) {
    if (!dnn || idx >= dnn->num_layers || !out) return;
    memcpy(out, dnn->layers[idx].params, sizeof(unsigned int) * NUM_PARAM_ELEMENTS);
}
extern "C" int aspen_b200_dnn_layer_type(aspen_dnn_t *dnn, unsigned int idx) {
    return (!dnn || idx >= dnn->num_layers) ? -1 : (int)dnn->layers[idx].type;
}
