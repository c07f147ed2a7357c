// Darknet-dialect .cfg reader: sections -> aspen_layer_t list with inferred shapes.
// Behaviour follows the reference parser (src/darknet_parser.c:339-575 for the file grammar and
// the key -> parameter mapping, src/input_parser.c:35-129 for the size inference); the code is a
// fresh std::string based implementation, not the Darknet list code the reference borrows.
#include "internal.h"

#include <fstream>
#include <utility>

namespace {

struct Section {
    std::string type;                                        // "[net]", "[convolutional]", ...
    std::vector<std::pair<std::string, std::string>> kv;    // in file order, first match wins
    const char *find(const char *key) const {
        for (auto &p : kv)
            if (p.first == key) return p.second.c_str();
        return nullptr;
    }
    int find_int(const char *key, int def) const {
        const char *v = find(key);
        return v ? atoi(v) : def;
    }
};

// Every blank is dropped, also inside a line ("filters = 64" == "filters=64"), darknet_parser.c:153-164.
std::string strip_blanks(const std::string &s) {
    std::string o;
    for (char c : s)
        if (c != ' ' && c != '\t' && c != '\n' && c != '\r') o.push_back(c);
    return o;
}

bool read_sections(const char *path, std::vector<Section> &out) {
    std::ifstream f(path);
    if (!f.is_open()) {
        ASPEN_ERR("Couldn't open file: %s\n", path);
        return false;
    }
    std::string raw;
    int line_no = 0;
    while (std::getline(f, raw)) {
        ++line_no;
        std::string line = strip_blanks(raw);
        if (line.empty() || line[0] == '#' || line[0] == ';') continue;
        if (line[0] == '[') {
            out.push_back(Section{line, {}});
            continue;
        }
        size_t eq = line.find('=');
        if (out.empty() || eq == std::string::npos || eq + 1 >= line.size()) {
            ASPEN_ERR("Config file error line %d, could parse: %s\n", line_no, line.c_str());
            continue;
        }
        out.back().kv.emplace_back(line.substr(0, eq), line.substr(eq + 1));
    }
    return true;
}

LAYER_TYPE section_layer_type(const std::string &t) {   // darknet_parser.c:408-436
    static const struct { const char *name; LAYER_TYPE type; } table[] = {
        {"[net]", INPUT_LAYER}, {"[network]", INPUT_LAYER},
        {"[conv]", CONV_LAYER}, {"[convolutional]", CONV_LAYER},
        {"[shortcut]", RESIDUAL_LAYER}, {"[batchnorm]", BATCHNORM_LAYER}, {"[yolo]", YOLO_LAYER},
        {"[activation]", ACTIVATION_LAYER}, {"[max]", MAXPOOL_LAYER}, {"[maxpool]", MAXPOOL_LAYER},
        {"[avg]", AVGPOOL_LAYER}, {"[avgpool]", AVGPOOL_LAYER}, {"[route]", ROUTE_LAYER},
        {"[conn]", FC_LAYER}, {"[connected]", FC_LAYER}, {"[soft]", SOFTMAX_LAYER},
        {"[softmax]", SOFTMAX_LAYER}, {"[append]", APPEND_LAYER}, {"[matmul]", MATMUL_LAYER},
        {"[attention_k]", K_ATTENTION_LAYER}, {"[attention_v]", V_ATTENTION_LAYER},
        {"[layernorm]", LAYERNORM_LAYER},
    };
    for (auto &e : table)
        if (t == e.name) return e.type;
    return NO_LAYER_TYPE;
}

LAYER_ACT activation_from_name(const char *s) {   // darknet_parser.c:390-406
    if (!s) return NO_ACTIVATION;
    static const struct { const char *name; LAYER_ACT act; } table[] = {
        {"logistic", SIGMOID}, {"linear", NO_ACTIVATION}, {"none", NO_ACTIVATION}, {"leaky", LEAKY_RELU},
        {"relu", RELU}, {"elu", ELU}, {"selu", SELU}, {"tanh", TANH}, {"gelu", GELU},
        {"gelu_acc", GELU_ACCURATE},
    };
    for (auto &e : table)
        if (strcmp(s, e.name) == 0) return e.act;
    ASPEN_ERR("Couldn't find activation function %s, going with ReLU\n", s);
    return RELU;
}

std::vector<float> parse_float_list(const char *s) {
    std::vector<float> v;
    while (s && *s) {
        v.push_back((float)atof(s));
        s = strchr(s, ',');
        if (s) ++s;
    }
    return v;
}

void fill_layer(const Section &s, aspen_layer_t *layer) {   // darknet_parser.c:455-552
    unsigned int *p = layer->params;
    layer->type = section_layer_type(s.type);
    p[IN_W] = s.find_int("width", 0);
    p[IN_H] = s.find_int("height", 0);
    p[IN_C] = s.find_int("channels", 0);
    p[WEIGHT_W] = p[WEIGHT_H] = s.find_int("size", 0);
    p[OUT_C] = s.find_int("filters", 0);
    if (p[OUT_C] == 0) p[OUT_C] = s.find_int("output", 0);
    p[STRIDE] = s.find_int("stride", 0);
    p[PADDING] = s.find_int("pad", 0);
    p[DILATION] = s.find_int("dilation", 0);
    p[MAT_M] = s.find_int("M", 0);
    p[MAT_N] = s.find_int("N", 0);
    p[MAT_K] = s.find_int("K", 0);
    p[NUM_HIDDEN] = s.find_int("n_embd", 0);
    p[NUM_HEAD] = s.find_int("n_head", 0);
    p[MASKED] = s.find_int("masked", 0);
    layer->activation = activation_from_name(s.find("activation"));
    int parent = s.find_int("parent", 0);
    if (layer->type == INPUT_LAYER)
        layer->parent_layers[PARENT_0] = nullptr;
    else
        layer->parent_layers[PARENT_0] = layer + (parent == 0 ? -1 : parent);
    int from = s.find_int("from", 0);
    if (from != 0) layer->parent_layers[PARENT_1] = layer + from;
    if (layer->type == YOLO_LAYER) {
        p[OUT_C] = s.find_int("classes", 0) + 5;
        std::vector<float> masks = parse_float_list(s.find("mask"));
        std::vector<float> anchors = parse_float_list(s.find("anchors"));
        if (masks.empty()) ASPEN_ERR("YOLO layer has no mask.\n");
        if (anchors.empty()) ASPEN_ERR("YOLO layer has no anchors.\n");
        unsigned int six[NUM_PARAM_ELEMENTS];
        for (auto &v : six) v = 6;
        LAYER_PARAMS order[] = {OUT_C};
        aspen_tensor_t *t = tensor_create(six, order, 1, layer->dnn->element_size);
        t->data = calloc(8, sizeof(float));
        for (int i = 0; i < 3 && i < (int)masks.size(); i++) {
            size_t a = (size_t)masks[i] * 2;
            if (a + 1 < anchors.size()) {
                ((float *)t->data)[i * 2] = anchors[a];
                ((float *)t->data)[i * 2 + 1] = anchors[a + 1];
            }
        }
        layer->tensors[ANCHOR_TENSOR] = t;
    }
}

unsigned int conv_out_extent(unsigned int in, unsigned int pad, unsigned int dil, unsigned int k, unsigned int stride) {
    return (in + 2 * pad - dil * (k - 1) - 1) / stride + 1;
}

bool infer_sizes(aspen_layer_t *layer) {   // input_parser.c:35-129
    unsigned int *p = layer->params;
    if (layer->type == INPUT_LAYER) {
        if (p[MAT_M] != 0) { p[OUT_H] = 1; p[OUT_W] = p[MAT_N]; p[OUT_C] = p[MAT_M]; }
        else { p[OUT_C] = p[IN_C]; p[OUT_H] = p[IN_H]; p[OUT_W] = p[IN_W]; }
        return true;
    }
    const unsigned int *pp = layer->parent_layers[PARENT_0]->params;
    p[IN_H] = pp[OUT_H]; p[IN_W] = pp[OUT_W]; p[IN_C] = pp[OUT_C];
    switch (layer->type) {
        case CONV_LAYER: case MAXPOOL_LAYER: case AVGPOOL_LAYER:
            if (p[STRIDE] == 0) p[STRIDE] = 1;
            if (p[DILATION] == 0) p[DILATION] = 1;
            p[OUT_H] = conv_out_extent(p[IN_H], p[PADDING], p[DILATION], p[WEIGHT_H], p[STRIDE]);
            p[OUT_W] = conv_out_extent(p[IN_W], p[PADDING], p[DILATION], p[WEIGHT_W], p[STRIDE]);
            if (layer->type != CONV_LAYER) p[OUT_C] = p[IN_C];
            return true;
        case SOFTMAX_LAYER: case FC_LAYER:
            p[OUT_H] = 1; p[OUT_W] = 1;
            return true;
        case RESIDUAL_LAYER:
            if (p[MAT_M] != 0) { p[OUT_H] = 1; p[OUT_W] = p[MAT_N]; p[OUT_C] = p[MAT_M]; }
            else { p[OUT_C] = p[IN_C]; p[OUT_H] = p[IN_H]; p[OUT_W] = p[IN_W]; }
            return true;
        case YOLO_LAYER:
            p[OUT_H] = 1;
            p[OUT_W] = p[IN_H] * p[IN_W] * (p[OUT_C] ? p[IN_C] / p[OUT_C] : 0);
            return true;
        case APPEND_LAYER:
            p[OUT_C] = p[IN_C] + layer->parent_layers[PARENT_1]->params[OUT_C];
            p[OUT_H] = p[IN_H] * p[STRIDE];
            p[OUT_W] = p[IN_W] * p[STRIDE];
            return true;
        case MATMUL_LAYER:
            p[MAT_K] = pp[MAT_M];
            return true;
        case V_ATTENTION_LAYER: case LAYERNORM_LAYER:
            return true;
        case K_ATTENTION_LAYER:
            p[MAT_K] = p[NUM_HEAD] ? p[NUM_HIDDEN] / p[NUM_HEAD] : 0;
            return true;
        default:
            ASPEN_ERR("ERROR: Unsupported layer type %s\n", layer_type_str[layer->type]);
            return false;
    }
}

}  // namespace

aspen_dnn_t *parse_cfg_file(const char *path) {
    const char *ext = strrchr(path, '.');
    if (!ext || strcmp(ext, ".cfg") != 0) {
        ASPEN_ERR("Input file type not supported: %s\n", path);
        return nullptr;
    }
    std::vector<Section> sections;
    if (!read_sections(path, sections) || sections.empty()) {
        ASPEN_ERR("Config file has no sections: %s\n", path);
        return nullptr;
    }
    std::vector<Section> kept;
    for (auto &s : sections) {
        if (section_layer_type(s.type) == NO_LAYER_TYPE)
            ASPEN_ERR("Unsupported section type: %s\n", s.type.c_str());
        else
            kept.push_back(std::move(s));
    }
    if (kept.empty() || section_layer_type(kept[0].type) != INPUT_LAYER) {
        ASPEN_ERR("First section must be [net] or [network]\n");
        return nullptr;
    }
    aspen_dnn_t *dnn = new aspen_dnn_t();
    strncpy(dnn->name, path, MAX_STRING_LEN - 1);
    dnn->num_layers = (unsigned int)kept.size();
    dnn->layers.resize(kept.size());
    for (size_t i = 0; i < kept.size(); i++) {
        dnn->layers[i].dnn = dnn;
        dnn->layers[i].layer_idx = (unsigned int)i;
    }
    for (size_t i = 0; i < kept.size(); i++) {
        fill_layer(kept[i], &dnn->layers[i]);
        aspen_layer_t *l = &dnn->layers[i];
        for (int pi = 0; pi < NUM_PARENT_ELEMENTS; pi++) {
            aspen_layer_t *par = l->parent_layers[pi];
            if (par && (par < dnn->layers.data() || par >= l)) {
                ASPEN_ERR("Layer %zu: parent reference out of range\n", i);
                delete dnn;
                return nullptr;
            }
        }
    }
    for (auto &l : dnn->layers)
        if (!infer_sizes(&l)) { delete dnn; return nullptr; }
    return dnn;
}
