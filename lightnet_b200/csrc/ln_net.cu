// Whole-network executor: the host side above the operators.  Mirrors the reference's
// GpuExecutableNetwork (lightnet-runtime/src/runtime/gpu_types.rs:220): build from a Darknet cfg
// (lightnet-model/src/cfg.rs:109, model.rs:3079), load Darknet weights (runtime/weights_io.rs:94),
// fold batch norm (weights_io.rs:32-92), walk the layers (gpu_forward_compact.rs:8), keep the
// convolution in front of a detection head at high precision (runtime/types.rs:146-170), and hand
// the heads to the device decode + NMS.
//
// f32 precision issues exactly the operator sequence of forward_compact through the f32 C ABI.
// 8-bit precisions run from a static plan: every layer output has a fixed home in device memory
// (sized for one micro-batch), multi-source routes are zero-copy where the producer can write into
// the concatenation buffer directly, and all tensor maps are built once.
#include <algorithm>
#include <cctype>
#include <cmath>
#include <fstream>
#include <memory>
#include <sstream>

#include "ln_conv_plan.h"

int ln_q_maxpool_launch(ln_ctx* ctx, int kind, const void* x, int64_t xs, void* y, int64_t ys, int64_t N, int C, int H, int W, int OH, int OW,
                        int size, int sx, int sy, int padding);
int ln_q_upsample_launch(ln_ctx* ctx, const void* x, int64_t xs, void* y, int64_t ys, int64_t N, int C, int H, int W, int stride);
int ln_q_copy_launch(ln_ctx* ctx, const void* x, int64_t xs, void* y, int64_t ys, int64_t pixels, int C);
int ln_q_upsample_requant_launch(ln_ctx* ctx, int kind, const void* x, int64_t xs, void* y, int64_t ys, int64_t N, int C, int H, int W, int stride, int reverse, float r);
int ln_q_shortcut_fit_launch(ln_ctx* ctx, const void* x, int64_t xs, int sc, int sh, int sw, void* y, int64_t ys, int64_t N, int C, int H, int W);
int ln_q_shortcut_launch(ln_ctx* ctx, int kind, const void* a, int64_t as, float sa, const void* b, int64_t bs, float sb, void* y, int64_t ys,
                         int64_t pixels, int C, int act, float inv_sy);
int ln_q_quantize_launch(ln_ctx* ctx, int kind, const float* x, void* y, int64_t N, int C, int H, int W, int64_t cstride, float inv_s);

namespace {

enum Kind { K_CONV = 0, K_MAXPOOL = 1, K_ROUTE = 2, K_SHORTCUT = 3, K_UPSAMPLE = 4, K_YOLO = 5 };

struct Shape4 { int w = 0, h = 0, c = 0, b = 0; };

struct QView {  // where a layer output lives in the 8-bit plan
    uint8_t* ptr = nullptr;
    int64_t cstride = 0;
    int c = 0, h = 0, w = 0;
    int buffer = -1;  // owning buffer index
};

struct NLayer {
    int kind = K_CONV;
    Shape4 in, out;
    int filters = 1, size = 1, stride_x = 1, stride_y = 1, dilation = 1, padding = 0, groups = 1;
    bool bn = false;
    int act = LN_ACT_LOGISTIC;
    std::vector<int> sources;
    int route_groups = 1, route_group_id = 0;
    int up_stride = 2;
    float up_scale = 1.0f;
    bool up_reverse = false;
    int classes = 20, num = 1;
    std::vector<int> mask;
    std::vector<float> anchors;
    float scale_x_y = 1.0f;
    bool new_coords = false;
    // anchor-free heads ([yolox] = 1, [ppyoloe] = 2, [yolonas] = 3; 0 = [yolo]): box entries per cell (model.rs:1086-1091)
    int modern = 0, modern_coords = 4;
    // host parameters (lightnet-layers/src/params.rs:7-26)
    std::vector<float> biases, scales, mean, var, weights;
    // device parameters
    ln_tensor* w_f32 = nullptr;  // BN-folded [F, C/g, k, k]
    ln_tensor* b_f32 = nullptr;  // folded bias [F]
    ln_conv_weights* wq = nullptr;
};

struct QStep {
    int layer = -1;
    int op = 0;  // 0 umma conv, 1 simt conv, 2 stem conv, 3 maxpool, 4 upsample, 5 copy, 6 shortcut, 7 quantize input, 8 shortcut fit, 9 requantising up-sample
    int sc = 0, sh = 0, sw = 0;  // shortcut fit: shape of the source
    ln_conv_umma_plan umma;
    ln_conv_geom geom;
    float2* mb = nullptr;
    bool head = false;          // output is an f32 head: pointer advances per micro-batch
    int head_index = -1;
    // glue
    const uint8_t* x = nullptr; int64_t xs = 0;
    const uint8_t* x2 = nullptr; int64_t xs2 = 0;
    uint8_t* y = nullptr; int64_t ys = 0;
    float sa = 1, sb = 1, inv_sy = 1;
    int C = 0, H = 0, W = 0, OH = 0, OW = 0;
    int pool_size = 0, pool_pad = 0;  // max-pool window actually run (a cascade shrinks it)
};

struct Section {
    std::string name;
    int line = 0;
    std::vector<std::pair<std::string, std::string>> kv;
    const std::string* find(const std::string& k) const {
        const std::string* r = nullptr;
        for (auto& e : kv) if (e.first == k) r = &e.second;  // last value wins (cfg.rs:155-157)
        return r;
    }
};

std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace((unsigned char)s[a])) ++a;
    while (b > a && std::isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
}
std::string lower(std::string s) {
    for (auto& c : s) c = (char)std::tolower((unsigned char)c);
    return s;
}

struct ParseError { std::string msg; };

long long get_i64(const Section& s, const char* k, long long d) {
    const std::string* v = s.find(k);
    if (!v) return d;
    try {
        size_t pos = 0;
        long long r = std::stoll(*v, &pos);
        if (pos != v->size()) throw 0;
        return r;
    } catch (...) { throw ParseError{"invalid integer \"" + *v + "\" for key " + k + " in [" + s.name + "] at line " + std::to_string(s.line)}; }
}
int get_usize(const Section& s, const char* k, int d) {
    long long v = get_i64(s, k, d);
    if (v < 0) throw ParseError{std::string("negative value for key ") + k + " in [" + s.name + "] at line " + std::to_string(s.line)};
    return (int)v;
}
float get_f32(const Section& s, const char* k, float d) {
    const std::string* v = s.find(k);
    if (!v) return d;
    try { return std::stof(*v); } catch (...) { throw ParseError{"invalid float \"" + *v + "\" for key " + k}; }
}
std::string get_str(const Section& s, const char* k, const char* d) {
    const std::string* v = s.find(k);
    return v ? *v : std::string(d);
}
template <class T>
std::vector<T> get_list(const Section& s, const char* k) {
    std::vector<T> out;
    const std::string* v = s.find(k);
    if (!v) return out;
    std::string item;
    auto flush = [&]() {
        if (item.empty()) return;
        try {
            if (std::is_floating_point<T>::value) out.push_back((T)std::stof(item));
            else out.push_back((T)std::stoll(item));
        } catch (...) { throw ParseError{"failed to parse list item \"" + item + "\" for key \"" + k + "\" in [" + s.name + "] at line " + std::to_string(s.line)}; }
        item.clear();
    };
    for (char ch : *v) {
        if (ch == ',' || std::isspace((unsigned char)ch)) flush();
        else item.push_back(ch);
    }
    flush();
    return out;
}

// ConfigFile::parse_str (lightnet-model/src/cfg.rs:109-171)
std::vector<Section> parse_sections(const std::string& text) {
    std::vector<Section> secs;
    std::istringstream in(text);
    std::string raw;
    int ln = 0;
    while (std::getline(in, raw)) {
        ++ln;
        size_t p = raw.find('#');
        if (p != std::string::npos) raw.resize(p);
        p = raw.find(';');
        if (p != std::string::npos) raw.resize(p);
        std::string line = trim(raw);
        if (line.empty()) continue;
        if (line.front() == '[' && line.back() == ']') {
            Section s;
            s.name = lower(trim(line.substr(1, line.size() - 2)));
            s.line = ln;
            secs.push_back(std::move(s));
            continue;
        }
        size_t eq = line.find('=');
        if (eq == std::string::npos) throw ParseError{"invalid config line " + std::to_string(ln) + ": expected key=value"};
        if (secs.empty()) throw ParseError{"encountered key/value before any section at line " + std::to_string(ln)};
        secs.back().kv.emplace_back(lower(trim(line.substr(0, eq))), trim(line.substr(eq + 1)));
    }
    if (secs.empty()) throw ParseError{"no Darknet sections found"};
    return secs;
}

int parse_activation(const std::string& s) {
    std::string a = lower(s);
    if (a == "linear") return LN_ACT_LINEAR;
    if (a == "logistic") return LN_ACT_LOGISTIC;
    if (a == "leaky") return LN_ACT_LEAKY;
    if (a == "mish") return LN_ACT_MISH;
    if (a == "swish") return LN_ACT_SWISH;
    if (a == "relu") return LN_ACT_RELU;
    throw ParseError{"activation \"" + s + "\" is not on the detector path"};
}

int conv_dim(int in, int pad, int size, int stride) {  // model.rs:6472
    int v = in + 2 * pad - size;
    if (v < 0) v = 0;
    return v / std::max(stride, 1) + 1;
}
int pool_dim(int in, int pad, int size, int stride) {  // model.rs:8854
    int v = in + pad - size;
    if (v < 0) v = 0;
    return v / std::max(stride, 1) + 1;
}
int resolve_relative(int layer_index, long long raw) {  // model.rs:6208
    long long a = raw < 0 ? layer_index + raw : raw;
    if (a < 0 || a >= layer_index) throw ParseError{"invalid route reference " + std::to_string(raw) + " at layer " + std::to_string(layer_index)};
    return (int)a;
}

__global__ void amax_f32_kernel(const float* __restrict__ x, int64_t n, unsigned* __restrict__ out) {
    float m = 0.0f;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = fabsf(x[i]);
        if (isfinite(v)) m = fmaxf(m, v);
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));  // non-negative floats order like their bits
}

}  // namespace

struct ln_net {
    ln_ctx* ctx = nullptr;
    int precision = LN_F32;
    int width = 0, height = 0, channels = 0, batch = 1;
    std::vector<NLayer> layers;
    bool weights_loaded = false;
    std::vector<float> scale;  // [0] input, [1+i] layer i output
    bool scales_set = false;
    int micro_batch = 0;
    // results of the last forward
    std::vector<ln_tensor*> out;       // f32 path: every layer output; 8-bit path: views (whole-batch runs only)
    std::vector<int> head_layers;      // indices of [yolo] layers
    std::vector<ln_tensor*> heads;     // f32 [batch, A*(5+classes), gh, gw]
    std::vector<ln_tensor*> modern_heads;  // per head: the activated (and box-decoded) tensor of an anchor-free head, else null
    // 8-bit plan
    bool plan_valid = false;
    int plan_mb = 0;
    std::vector<QStep> steps;
    std::vector<std::pair<void*, size_t>> buffers;
    std::vector<QView> views;
    ln_tensor* input_dev = nullptr;    // staging for host inputs
    // Host-input pipeline of the 8-bit path: two part-batch networks (a quarter and three quarters of the batch) with the same
    // weights and scales; the upload of the second part overlaps the layers of the first (copy engine + its own stream), each
    // part decodes its own images.
    std::string cfg_text;
    bool host_pipeline = true;
    ln_net* pipe[2] = {nullptr, nullptr};
    std::vector<ln_tensor*> pipe_heads;  // whole-batch head tensors the two part networks write their image ranges of
    std::vector<ln_tensor*> ext_heads;   // part network: its views into the owner's pipe_heads (used instead of own head storage)
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t copy_ev[2] = {nullptr, nullptr};
    // ln_net_submit / ln_net_collect: two input slots; `submitted` counts uploads enqueued, `collected` batches run
    ln_tensor* slot_dev[2] = {nullptr, nullptr};
    cudaEvent_t slot_ev[2] = {nullptr, nullptr};
    void* slot_staging[2] = {nullptr, nullptr};  // 8-bit pixels + metadata of ln_net_submit_u8, back to the pool at collect
    size_t slot_staging_bytes[2] = {0, 0};
    long long submitted = 0, collected = 0;
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    float times_ms[2] = {0, 0};
    // CUDA graph of the 8-bit plan (one graph = the whole batch: every micro-batch, every layer)
    bool fuse_shortcut = true;  // a linear [shortcut] whose input is a convolution nobody else reads runs in that convolution's epilogue
    std::vector<char> fused_into_next;  // per layer (8-bit plan): 1 = runs in the next layer's shortcut epilogue, no output; 2 = output kept in space-to-depth layout
    bool use_graph = true;
    // One graph per (input pointer, epilogue mode): a caller that alternates between a few input tensors (the two slots of
    // ln_net_submit) replays a graph for each.  A key runs eagerly the first time it is seen and is captured the second time, so a
    // caller whose input pointer changes on every call pays no capture; the least recently used entry makes room.
    struct GraphSlot {
        const void* input = nullptr;
        bool exact = false;
        cudaGraphExec_t exec = nullptr;
        unsigned long long used = 0;
    };
    GraphSlot graphs[4];
    unsigned long long graph_clock = 0;
    // optional per-launch timing
    bool profile = false;
    std::vector<cudaEvent_t> prof_events;
    std::vector<float> prof_layer_ms;
    float prof_op_ms[8] = {0};
    int prof_op_launches[8] = {0};
};

namespace {

void build_layers(ln_net* net, const std::string& cfg, int batch_override) {
    auto secs = parse_sections(cfg);
    const Section& n = secs[0];
    if (n.name != "net" && n.name != "network") throw ParseError{"the first section must be [net]"};
    net->width = get_usize(n, "width", 0);
    net->height = get_usize(n, "height", 0);
    net->channels = get_usize(n, "channels", 0);
    int subdiv = std::max(get_usize(n, "subdivisions", 1), 1), ts = std::max(get_usize(n, "time_steps", 1), 1);
    net->batch = get_usize(n, "batch", 1) / subdiv * ts;  // model.rs:247-249
    if (batch_override > 0) net->batch = batch_override;  // model.rs:3256
    if (net->width < 1 || net->height < 1 || net->channels < 1 || net->batch < 1) throw ParseError{"[net] needs positive width, height, channels and batch"};
    Shape4 cur;
    cur.w = net->width; cur.h = net->height; cur.c = net->channels; cur.b = net->batch;
    for (size_t si = 1; si < secs.size(); ++si) {
        const Section& s = secs[si];
        const int li = (int)net->layers.size();
        NLayer L;
        L.in = cur;
        if (s.name == "conv" || s.name == "convolutional") {  // model.rs:4088-4144
            L.kind = K_CONV;
            int stride = get_usize(s, "stride", 1);
            L.size = get_usize(s, "size", 1);
            L.padding = get_i64(s, "pad", 0) != 0 ? L.size / 2 : get_usize(s, "padding", 0);
            L.filters = get_usize(s, "filters", 1);
            L.groups = get_usize(s, "groups", 1);
            L.stride_x = get_usize(s, "stride_x", stride);
            L.stride_y = get_usize(s, "stride_y", stride);
            L.dilation = get_usize(s, "dilation", 1);
            L.bn = get_i64(s, "batch_normalize", 0) != 0;
            L.act = parse_activation(get_str(s, "activation", "logistic"));
            if (L.groups < 1 || L.filters % L.groups || cur.c % L.groups) throw ParseError{"convolution groups do not divide filters / channels at layer " + std::to_string(li)};
            L.out.w = conv_dim(cur.w, L.padding, L.size, L.stride_x);
            L.out.h = conv_dim(cur.h, L.padding, L.size, L.stride_y);
            L.out.c = L.filters;
            L.out.b = cur.b;
            L.biases.assign(L.filters, 0.0f);
            L.weights.assign((size_t)L.filters * (cur.c / L.groups) * L.size * L.size, 0.0f);
            if (L.bn) { L.scales.assign(L.filters, 1.0f); L.mean.assign(L.filters, 0.0f); L.var.assign(L.filters, 1.0f); }
        } else if (s.name == "max" || s.name == "maxpool") {  // model.rs:4165-4183
            L.kind = K_MAXPOOL;
            int stride = get_usize(s, "stride", 1);
            L.size = get_usize(s, "size", stride);
            L.stride_x = get_usize(s, "stride_x", stride);
            L.stride_y = get_usize(s, "stride_y", stride);
            L.padding = get_usize(s, "padding", L.size > 0 ? L.size - 1 : 0);
            if (get_i64(s, "maxpool_depth", 0) != 0) throw ParseError{"maxpool_depth is not on the detector path"};
            L.out.w = pool_dim(cur.w, L.padding, L.size, L.stride_x);
            L.out.h = pool_dim(cur.h, L.padding, L.size, L.stride_y);
            L.out.c = cur.c; L.out.b = cur.b;
        } else if (s.name == "route") {  // model.rs:4225-4229, :6138
            L.kind = K_ROUTE;
            auto raw = get_list<long long>(s, "layers");
            if (raw.empty()) throw ParseError{"route layer #" + std::to_string(li) + " must list at least one source layer"};
            L.route_groups = std::max(get_usize(s, "groups", 1), 1);
            L.route_group_id = get_usize(s, "group_id", 0);
            int ch = 0;
            Shape4 first;
            for (size_t k = 0; k < raw.size(); ++k) {
                int src = resolve_relative(li, raw[k]);
                L.sources.push_back(src);
                const Shape4& sh = net->layers[src].out;
                if (k == 0) first = sh;
                else if (sh.w != first.w || sh.h != first.h) throw ParseError{"route layer #" + std::to_string(li) + " mixes incompatible spatial shapes"};
                ch += sh.c;
            }
            L.out.w = first.w; L.out.h = first.h; L.out.c = ch / L.route_groups; L.out.b = cur.b;
        } else if (s.name == "shortcut") {  // model.rs:4230-4237
            L.kind = K_SHORTCUT;
            for (auto r : get_list<long long>(s, "from")) L.sources.push_back(resolve_relative(li, r));
            L.act = parse_activation(get_str(s, "activation", "linear"));
            L.out = cur;
        } else if (s.name == "upsample") {  // model.rs:4263-4270, :5711-5733
            L.kind = K_UPSAMPLE;
            long long st = get_i64(s, "stride", 2);
            L.up_reverse = st < 0;
            L.up_stride = (int)std::llabs(st);
            if (L.up_stride == 0) throw ParseError{"upsample layer #" + std::to_string(li) + " cannot use stride=0"};
            L.up_scale = get_f32(s, "scale", 1.0f);
            L.out = cur;
            if (L.up_reverse) { L.out.w = cur.w / L.up_stride; L.out.h = cur.h / L.up_stride; }
            else { L.out.w = cur.w * L.up_stride; L.out.h = cur.h * L.up_stride; }
        } else if (s.name == "yolo" || s.name == "gaussian_yolo") {  // model.rs:4271-4344, :4513-4543
            // at inference [gaussian_yolo] is the same identity layer with the same spec, decoded by the same function
            // (detect.rs:78, :135); its num is max(len(mask), num)
            L.kind = K_YOLO;
            L.mask = get_list<int>(s, "mask");
            L.num = get_usize(s, "num", L.mask.empty() ? 1 : (int)L.mask.size());
            if (s.name == "gaussian_yolo" && L.num < (int)L.mask.size()) L.num = (int)L.mask.size();
            if (L.mask.empty()) for (int k = 0; k < L.num; ++k) L.mask.push_back(k);
            L.classes = get_usize(s, "classes", 20);
            L.anchors = get_list<float>(s, "anchors");
            L.scale_x_y = get_f32(s, "scale_x_y", 1.0f);
            L.new_coords = get_i64(s, "new_coords", 0) != 0;
            for (int m : L.mask)  // detection_geometry.rs:80-95 anchor_pair
                if ((size_t)(2 * m + 1) >= L.anchors.size()) throw ParseError{"missing anchor for YOLO mask index " + std::to_string(m)};
            if (L.mask.size() > 8) throw ParseError{"more than 8 anchors per head"};
            L.out = cur;
            net->head_layers.push_back(li);
        } else if (s.name == "yolox" || s.name == "ppyoloe" || s.name == "yolonas") {  // model.rs:4835-4842, :8818-8852 parse_modern_yolo_spec
            // an anchor-free head: its forward is the output activation (lib.rs:4884); the distribution heads are then decoded to
            // final boxes on the device (lib.rs:4936), so the head tensor has 5 + classes channels for every kind
            L.kind = K_YOLO;
            L.modern = s.name == "yolox" ? 1 : (s.name == "ppyoloe" ? 2 : 3);
            L.classes = get_usize(s, "classes", 20);
            if (L.classes == 0) throw ParseError{"[yolox] at line " + std::to_string(s.line) + ": classes must be > 0"};
            if (get_usize(s, "max", 200) == 0) throw ParseError{"[yolox] at line " + std::to_string(s.line) + ": max must be > 0"};
            const int reg_max = (int)get_usize(s, "reg_max", 16);
            L.modern_coords = L.modern == 1 ? 4 : 4 * ((reg_max < 1 ? 1 : (reg_max > 64 ? 64 : reg_max)) + 1);
            if (cur.c != L.modern_coords + 1 + L.classes)
                throw ParseError{"[" + s.name + "] at line " + std::to_string(s.line) + ": the layer before it has " + std::to_string(cur.c) + " channels, the head needs " +
                                 std::to_string(L.modern_coords + 1 + L.classes)};
            L.mask = {0};
            L.num = 1;
            L.anchors = {1.0f, 1.0f};
            L.out = cur;
            L.out.c = 5 + L.classes;
            net->head_layers.push_back(li);
        } else {
            throw ParseError{"layer [" + s.name + "] at line " + std::to_string(s.line) + " is not on the detector path"};
        }
        cur = L.out;
        net->layers.push_back(std::move(L));
    }
}

bool feeds_head(const ln_net* net, int i) {  // runtime/types.rs:146-170
    return net->layers[i].kind == K_CONV && i + 1 < (int)net->layers.size() && net->layers[i + 1].kind == K_YOLO;
}

void release_outputs(ln_net* net) {
    for (auto*& t : net->out) { ln_tensor_release(t); t = nullptr; }
    net->out.clear();
}
void release_heads(ln_net* net) {
    for (auto*& t : net->heads) { ln_tensor_release(t); t = nullptr; }
    net->heads.clear();
    for (auto*& t : net->modern_heads) { if (t) ln_tensor_release(t); t = nullptr; }
    net->modern_heads.clear();
}
void release_graph(ln_net* net) {
    for (auto& g : net->graphs) {
        if (g.exec) cudaGraphExecDestroy(g.exec);
        g = ln_net::GraphSlot();
    }
}

void release_plan(ln_net* net) {
    ln_ctx* ctx = net->ctx;
    release_graph(net);
    for (auto& s : net->steps) {
        if (s.mb) ln_pool_free(ctx, s.mb, (size_t)net->layers[s.layer].wq->fpad * sizeof(float2));
        ln_conv_umma_plan_release(ctx, &s.umma);
    }
    net->steps.clear();
    for (auto& b : net->buffers) ln_pool_free(ctx, b.first, b.second);
    net->buffers.clear();
    net->views.clear();
    net->plan_valid = false;
}

// ---- f32 forward: the operator sequence of forward_compact (gpu_forward_compact.rs:8-540) --------
int forward_f32(ln_net* net, const ln_tensor* input, unsigned* amax_dev) {
    ln_ctx* ctx = net->ctx;
    release_outputs(net);
    release_heads(net);
    const int NL = (int)net->layers.size();
    net->out.assign(NL, nullptr);
    auto record_amax = [&](const ln_tensor* t, int slot) {
        if (!amax_dev) return;
        int64_t n = t->count();
        int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)ctx->sm_count * 8);
        amax_f32_kernel<<<grid, 256, 0, ctx->stream>>>((const float*)t->ptr, n, amax_dev + slot);
        ctx->launches++;
    };
    record_amax(input, 0);
    for (int i = 0; i < NL; ++i) {
        NLayer& L = net->layers[i];
        const ln_tensor* x = i == 0 ? input : net->out[i - 1];
        const int64_t oshape[4] = {L.out.b, L.out.c, L.out.h, L.out.w};
        ln_tensor* y = nullptr;
        int rc = LN_OK;
        switch (L.kind) {
            case K_CONV: {  // layers/convolutional/gpu.rs:138-209: conv2d_f32_with_precision + bias_activation_f32
                ln_tensor* conv = nullptr;
                rc = ln_conv2d_f32(ctx, x, L.w_f32, oshape, L.in.c, L.in.h, L.in.w, L.filters, L.size, L.stride_x, L.stride_y, L.dilation, L.padding,
                                   L.groups, &conv);
                if (rc == LN_OK) rc = ln_bias_activation_f32(ctx, conv, L.b_f32, L.filters, (int64_t)L.out.h * L.out.w, L.act, &y);
                ln_tensor_release(conv);
                break;
            }
            case K_MAXPOOL:  // layers/pool/gpu.rs:13-42
                rc = ln_maxpool_f32(ctx, x, oshape, L.in.c, L.in.h, L.in.w, L.size, L.stride_x, L.stride_y, L.padding, &y);
                break;
            case K_ROUTE: {  // layers/route/gpu.rs:61-108
                std::vector<const ln_tensor*> ins;
                std::vector<int64_t> offs, chans, totals;
                for (int src : L.sources) {
                    const ln_tensor* t = net->out[src];
                    int64_t chunk = t->c / L.route_groups;
                    ins.push_back(t);
                    offs.push_back(chunk * L.route_group_id);
                    chans.push_back(chunk);
                    totals.push_back(t->c);
                }
                rc = ln_route_concat_f32(ctx, ins.data(), (int)ins.size(), offs.data(), chans.data(), totals.data(), oshape, (int64_t)L.out.h * L.out.w, &y);
                break;
            }
            case K_SHORTCUT: {  // layers/shortcut/gpu.rs:153-213: fit? + add per source, then activation
                ln_tensor* acc = const_cast<ln_tensor*>(x);
                ln_tensor_retain(acc);
                for (int src : L.sources) {
                    const ln_tensor* s = net->out[src];
                    ln_tensor* fitted = nullptr;
                    if (s->n != acc->n) { rc = ln_fail(ctx, LN_ERR_SHAPE, "shortcut layer #%d mixes incompatible batch shapes", i); break; }
                    if (s->count() != acc->count()) {
                        rc = ln_shortcut_fit_f32(ctx, s, L.out.b, oshape, &fitted);
                        if (rc) break;
                        s = fitted;
                    }
                    ln_tensor* sum = nullptr;
                    rc = ln_shortcut_add_f32(ctx, acc, s, &sum);
                    ln_tensor_release(fitted);
                    if (rc) break;
                    ln_tensor_release(acc);
                    acc = sum;
                }
                if (rc == LN_OK) rc = ln_activation_f32(ctx, acc, L.act, &y);
                ln_tensor_release(acc);
                break;
            }
            case K_UPSAMPLE:  // layers/upsample/gpu.rs:12-33
                rc = ln_upsample_f32(ctx, x, oshape, L.in.c, L.in.h, L.in.w, L.up_stride, L.up_scale, L.up_reverse ? 1 : 0, &y);
                break;
            case K_YOLO:  // gpu_forward_compact.rs:420-429: clone the handle, mark the head
                y = const_cast<ln_tensor*>(x);
                ln_tensor_retain(y);
                net->heads.push_back(y);
                ln_tensor_retain(y);
                break;
        }
        if (rc) return rc;
        net->out[i] = y;
        record_amax(y, i + 1);
    }
    return LN_OK;
}

// ---- binary16 forward: the operator sequence of forward_compact_f16 (gpu_f16.rs:21-957) over the F16 twin ------------------
// Every convolution, the ones in front of the heads included, runs conv2d_bias_act_f16 on cached conv_weights_f16
// (gpu_f16.rs:164-224); shortcuts fit mismatched sources and add them one by one, the layer's activation going to the last
// add (:440-490); a [yolo] layer hands the previous output on, widened to f32 as download_f16 does for the decoder (:898-925).
int forward_f16(ln_net* net, const ln_tensor* input) {
    ln_ctx* ctx = net->ctx;
    release_outputs(net);
    release_heads(net);
    const int NL = (int)net->layers.size();
    net->out.assign(NL, nullptr);
    ln_tensor* in16 = nullptr;
    int rc = ln_tensor_narrow_f16(ctx, input, &in16);  // upload_f16: the f32 input rounded to binary16 on the device
    if (rc) return rc;
    for (int i = 0; i < NL && rc == LN_OK; ++i) {
        NLayer& L = net->layers[i];
        const ln_tensor* x = i == 0 ? in16 : net->out[i - 1];
        const int64_t oshape[4] = {L.out.b, L.out.c, L.out.h, L.out.w};
        ln_tensor* y = nullptr;
        switch (L.kind) {
            case K_CONV:
                rc = ln_conv2d_bias_act_f16(ctx, x, L.wq, L.b_f32, oshape, L.in.c, L.in.h, L.in.w, L.filters, L.size, L.stride_x, L.stride_y, L.dilation, L.padding,
                                            L.groups, L.act, &y);
                break;
            case K_MAXPOOL:
                rc = ln_maxpool_f16(ctx, x, oshape, L.in.c, L.in.h, L.in.w, L.size, L.stride_x, L.stride_y, L.padding, &y);
                break;
            case K_ROUTE: {
                std::vector<const ln_tensor*> ins;
                std::vector<int64_t> offs, chans, totals;
                for (int src : L.sources) {
                    const ln_tensor* t = net->out[src];
                    const int64_t chunk = t->c / L.route_groups;
                    ins.push_back(t);
                    offs.push_back(chunk * L.route_group_id);
                    chans.push_back(chunk);
                    totals.push_back(t->c);
                }
                rc = ln_route_concat_f16(ctx, ins.data(), (int)ins.size(), offs.data(), chans.data(), totals.data(), oshape, (int64_t)L.out.h * L.out.w, &y);
                break;
            }
            case K_SHORTCUT: {
                ln_tensor* acc = const_cast<ln_tensor*>(x);
                ln_tensor_retain(acc);
                for (size_t k = 0; k < L.sources.size() && rc == LN_OK; ++k) {
                    const ln_tensor* s = net->out[L.sources[k]];
                    ln_tensor* fitted = nullptr;
                    if (s->n != acc->n) { rc = ln_fail(ctx, LN_ERR_SHAPE, "shortcut layer #%d mixes incompatible batch shapes", i); break; }
                    if (s->c != acc->c || s->h != acc->h || s->w != acc->w) {
                        rc = ln_shortcut_fit_f16(ctx, s, L.out.b, oshape, &fitted);
                        if (rc) break;
                        s = fitted;
                    }
                    ln_tensor* sum = nullptr;
                    rc = ln_shortcut_add_act_f16(ctx, acc, s, k + 1 == L.sources.size() ? L.act : LN_ACT_LINEAR, &sum);
                    ln_tensor_release(fitted);
                    if (rc) break;
                    ln_tensor_release(acc);
                    acc = sum;
                }
                if (rc == LN_OK) y = acc;
                else ln_tensor_release(acc);
                break;
            }
            case K_UPSAMPLE:
                rc = ln_upsample_f16(ctx, x, oshape, L.in.c, L.in.h, L.in.w, L.up_stride, L.up_scale, L.up_reverse ? 1 : 0, &y);
                break;
            case K_YOLO: {
                y = const_cast<ln_tensor*>(x);
                ln_tensor_retain(y);
                ln_tensor* head = nullptr;
                rc = ln_tensor_widen_f16(ctx, x, &head);
                if (rc == LN_OK) net->heads.push_back(head);
                break;
            }
        }
        if (rc == LN_OK) net->out[i] = y;
        else ln_tensor_release(y);
    }
    ln_tensor_release(in16);
    return rc;
}

// ---- per-tensor scales from the calibration amax (tensors joined by route / maxpool / upsample share one)
void scales_from_amax(ln_net* net, const std::vector<float>& amax, float qmax) {
    const int T = (int)net->layers.size() + 1;
    std::vector<int> parent(T);
    for (int t = 0; t < T; ++t) parent[t] = t;
    auto find = [&](int a) { while (parent[a] != a) a = parent[a] = parent[parent[a]]; return a; };
    auto join = [&](int a, int b) { a = find(a); b = find(b); if (a != b) parent[std::max(a, b)] = std::min(a, b); };
    for (int i = 0; i < T - 1; ++i) {
        const NLayer& L = net->layers[i];
        // tensors whose codes are copied share a scale; an up-sample that scales or sums (reverse) requantises instead
        if (L.kind == K_MAXPOOL || L.kind == K_YOLO || (L.kind == K_UPSAMPLE && !L.up_reverse && L.up_scale == 1.0f)) join(i + 1, i);
        if (L.kind == K_ROUTE) for (int s : L.sources) join(i + 1, s + 1);
    }
    std::vector<float> gmax(T, 0.0f);
    for (int t = 0; t < T; ++t) { int r = find(t); gmax[r] = std::max(gmax[r], amax[t]); }
    net->scale.assign(T, 1.0f);
    for (int t = 0; t < T; ++t) {
        float m = gmax[find(t)];
        net->scale[t] = (m > 0.0f && std::isfinite(m)) ? m / qmax : 1.0f;
    }
    net->scales_set = true;
}

// ---- 8-bit plan ----------------------------------------------------------------------------------
int build_plan(ln_net* net, int mb) {
    ln_ctx* ctx = net->ctx;
    release_plan(net);
    const int NL = (int)net->layers.size();
    const int kind = net->precision == LN_F8 ? LN_KIND_F8 : LN_KIND_I8;
    if (!net->scales_set) return ln_fail(ctx, LN_ERR_ARG, "8-bit forward needs per-tensor scales: call ln_net_calibrate or ln_net_set_scales first");
    // 1. support checks
    for (int i = 0; i < NL; ++i) {
        const NLayer& L = net->layers[i];
        if (L.kind == K_CONV && (L.dilation != 1 || L.stride_x != L.stride_y))
            return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d: 8-bit convolution needs dilation=1, stride_x=stride_y", i);
        if (L.kind == K_CONV && L.groups != 1 && i == 0) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #0: the first layer cannot be a grouped convolution in the 8-bit plan");
        if (L.kind == K_UPSAMPLE && !(L.up_scale > 0.0f)) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d: 8-bit up-sample needs a positive scale", i);
        if (L.kind == K_SHORTCUT && L.sources.size() != 1) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d: 8-bit shortcut takes exactly one source", i);
        if (L.kind == K_YOLO && (i == 0 || !feeds_head(net, i - 1))) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d: [yolo] must follow a convolution", i);
        if (L.kind == K_ROUTE && L.route_groups > 1 && (L.sources.size() != 1)) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d: grouped route with several sources", i);
        if (L.kind != K_CONV && L.kind != K_YOLO && i > 0 && feeds_head(net, i - 1)) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d reads a head convolution's f32 output", i);
        if (L.kind == K_ROUTE || L.kind == K_SHORTCUT)
            for (int s : L.sources)
                if (feeds_head(net, s) || net->layers[s].kind == K_YOLO) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d reads a head's f32 output", i);
    }
    // 2. homes: alias chains and zero-copy concatenation
    std::vector<int> alias(NL, -1);        // single-source ungrouped route -> its source
    std::vector<int> home_buf(NL, -1);     // layer output placed inside another layer's (route) buffer
    std::vector<int> home_off(NL, 0);
    auto root_of = [&](int l) { while (alias[l] >= 0) l = alias[l]; return l; };
    for (int i = 0; i < NL; ++i) {
        const NLayer& L = net->layers[i];
        if (L.kind == K_ROUTE && L.sources.size() == 1 && L.route_groups == 1) alias[i] = L.sources[0];
    }
    for (int i = 0; i < NL; ++i) {
        const NLayer& L = net->layers[i];
        if (L.kind != K_ROUTE || L.sources.size() < 2) continue;
        int off = 0;
        for (int s : L.sources) {
            const int r = root_of(s);
            const NLayer& P = net->layers[r];
            const bool producer = (P.kind == K_CONV && !feeds_head(net, r)) || P.kind == K_SHORTCUT || P.kind == K_MAXPOOL || P.kind == K_UPSAMPLE;
            if (producer && home_buf[r] < 0 && off % 32 == 0 && P.out.c % 32 == 0) { home_buf[r] = i; home_off[r] = off; }
            off += net->layers[s].out.c;
        }
    }
    // 2b. shortcut fusion: conv i -> shortcut i+1 (linear, one same-shape source), conv output read by nobody else
    net->fused_into_next.assign(NL, 0);
    if (net->fuse_shortcut && kind == LN_KIND_I8) {
        std::vector<int> readers(NL, 0);
        for (int i = 0; i < NL; ++i) {
            if (i > 0 && net->layers[i].kind != K_ROUTE) readers[i - 1]++;  // sequential input (a route ignores it)
            if (net->layers[i].kind == K_ROUTE || net->layers[i].kind == K_SHORTCUT)
                for (int s : net->layers[i].sources) readers[s]++;
        }
        for (int i = 1; i + 1 < NL; ++i) {
            const NLayer& C = net->layers[i];
            const NLayer& S = net->layers[i + 1];
            if (C.kind != K_CONV || S.kind != K_SHORTCUT || S.act != LN_ACT_LINEAR || S.sources.size() != 1) continue;
            { const Shape4& ss = net->layers[S.sources[0]].out; if (ss.w != S.out.w || ss.h != S.out.h || ss.c != S.out.c) continue; }  // a fitted source is not fused
            if (readers[i] != 1 || S.sources[0] == i || C.filters % 32 != 0 || feeds_head(net, i)) continue;
            if (!ln_conv_umma_supported(ln_round_up(C.in.c, 32), C.size, C.stride_x, C.stride_y, C.dilation, C.groups, C.in.w, C.in.h)) continue;
            net->fused_into_next[i] = 1;
        }
    }
    // 2c. the first layer writes the 2x2 space-to-depth image of its 32 channels when its only reader is a 3x3 stride-2 convolution:
    // that convolution then reads 4 taps of 128-byte rows instead of 9 taps of 32-byte rows (value 2 = "kept in another layout")
    if (net->fuse_shortcut && NL > 1) {
        const NLayer& A = net->layers[0];
        const NLayer& B = net->layers[1];
        int readers0 = 0;
        for (int i = 1; i < NL; ++i) {
            if (i == 1 && net->layers[i].kind != K_ROUTE) readers0++;
            if (net->layers[i].kind == K_ROUTE || net->layers[i].kind == K_SHORTCUT)
                for (int s : net->layers[i].sources) readers0 += s == 0;
        }
        if (A.kind == K_CONV && A.in.c == 3 && A.size == 3 && A.filters == 32 && A.groups == 1 && A.out.w % 2 == 0 && A.out.h % 2 == 0 && !feeds_head(net, 0) &&
            B.kind == K_CONV && B.size == 3 && B.stride_x == 2 && B.stride_y == 2 && B.padding == 1 && B.groups == 1 && B.dilation == 1 && readers0 == 1 &&
            !net->fused_into_next[1] && !feeds_head(net, 1))
            net->fused_into_next[0] = 2;
    }
    // 3. buffers and views
    net->views.assign(NL, QView());
    std::vector<int> buffer_of(NL, -1);
    auto alloc_buffer = [&](int64_t bytes) -> int {
        void* p = ln_pool_alloc(ctx, (size_t)bytes);
        if (!p) return -1;
        cudaMemsetAsync(p, 0, (size_t)bytes, ctx->stream);
        net->buffers.emplace_back(p, (size_t)bytes);
        return (int)net->buffers.size() - 1;
    };
    for (int i = 0; i < NL; ++i) {  // routes with several sources own a concatenation buffer; allocate those first
        const NLayer& L = net->layers[i];
        if (L.kind == K_ROUTE && L.sources.size() >= 2) {
            int64_t cs = ln_round_up(L.out.c, 32);
            int b = alloc_buffer((int64_t)mb * L.out.h * L.out.w * cs);
            if (b < 0) return LN_ERR_CUDA;
            buffer_of[i] = b;
            QView v;
            v.ptr = (uint8_t*)net->buffers[b].first; v.cstride = cs; v.c = L.out.c; v.h = L.out.h; v.w = L.out.w; v.buffer = b;
            net->views[i] = v;
        }
    }
    for (int i = 0; i < NL; ++i) {
        const NLayer& L = net->layers[i];
        QView v;
        v.c = L.out.c; v.h = L.out.h; v.w = L.out.w;
        if (L.kind == K_YOLO || feeds_head(net, i)) { net->views[i] = v; continue; }  // f32 heads live elsewhere
        if (L.kind == K_ROUTE) {
            if (L.sources.size() >= 2) continue;  // done above
            if (alias[i] >= 0) { net->views[i] = net->views[root_of(i)]; continue; }
            // grouped single-source route: a channel slice of the source
            const QView& sv = net->views[L.sources[0]];
            const int chunk = net->layers[L.sources[0]].out.c / L.route_groups, start = chunk * L.route_group_id;
            if (start % 16 == 0) {
                v = sv; v.c = chunk; v.ptr = sv.ptr + start;
                net->views[i] = v;
                continue;
            }
            // unaligned slice: gets its own buffer and a copy step (below)
        }
        if (home_buf[i] >= 0) {
            const QView& hv = net->views[home_buf[i]];
            v.ptr = hv.ptr + home_off[i]; v.cstride = hv.cstride; v.buffer = hv.buffer;
        } else {
            int64_t cs = ln_round_up(L.out.c, 32);
            int b = alloc_buffer((int64_t)mb * L.out.h * L.out.w * cs);
            if (b < 0) return LN_ERR_CUDA;
            v.ptr = (uint8_t*)net->buffers[b].first; v.cstride = cs; v.buffer = b;
        }
        net->views[i] = v;
    }
    // 4. heads
    release_heads(net);
    for (size_t k = 0; k < net->head_layers.size(); ++k) {
        const NLayer& L = net->layers[net->head_layers[k]];
        ln_tensor* t;
        if (net->ext_heads.size() == net->head_layers.size()) {  // a part network of the host-input pipeline writes into its owner's heads
            t = net->ext_heads[k];
            ln_tensor_retain(t);
        } else {
            t = ln_tensor_new(ctx, LN_F32, net->batch, L.modern ? L.modern_coords + 1 + L.classes : L.out.c, L.out.h, L.out.w);  // what the convolution writes
        }
        if (!t) return LN_ERR_CUDA;
        net->heads.push_back(t);
    }
    // 5. steps
    int head_counter = 0;
    for (int i = 0; i < NL; ++i) {
        NLayer& L = net->layers[i];
        const float sx = net->scale[i], sy = net->scale[i + 1];
        QStep st;
        st.layer = i;
        switch (L.kind) {
            case K_CONV: {
                const bool head = feeds_head(net, i);
                st.head = head;
                if (head) st.head_index = head_counter++;
                st.mb = (float2*)ln_pool_alloc(ctx, (size_t)L.wq->fpad * sizeof(float2));
                if (!st.mb) return LN_ERR_CUDA;
                int rc = ln_conv_umma_make_mb(ctx, L.wq->wscale, (const float*)L.b_f32->ptr, sx, L.filters, (int)L.wq->fpad, st.mb);
                if (rc) return rc;
                ln_conv_geom& g = st.geom;
                g.kind = kind;
                g.N = mb; g.H = L.in.h; g.W = L.in.w; g.C = L.in.c; g.cpad = (int)L.wq->cpad;
                g.w = L.wq->w; g.F = L.filters; g.fpad = (int)L.wq->fpad; g.k = L.size; g.stride = L.stride_x; g.pad = L.padding;
                g.OH = L.out.h; g.OW = L.out.w; g.act = L.act;
                g.out_kind = head ? LN_OUT_F32 : LN_OUT_Q;
                g.inv_sy = head ? 1.0f : 1.0f / sy;
                g.small_acc = kind == LN_KIND_I8 && 127.0f * L.wq->max_l1 < 4194304.0f;
                g.acc_shift = kind == LN_KIND_I8 && !head ? ln_acc_shift(L.wq->max_l1, sx, L.wq->max_scale, g.inv_sy) : -1;
                if (head) { g.out = net->heads[st.head_index]->ptr; g.out_pixel_stride = 0; }
                else if (net->fused_into_next[i] == 1) {
                    const int sl = i + 1, src = net->layers[sl].sources[0];
                    g.out = net->views[sl].ptr; g.out_pixel_stride = net->views[sl].cstride;
                    g.res = net->views[src].ptr; g.res_pixel_stride = net->views[src].cstride;
                    g.s_c = sy; g.s_res = net->scale[src + 1]; g.inv_sy2 = 1.0f / net->scale[sl + 1];
                }
                else { g.out = net->views[i].ptr; g.out_pixel_stride = net->views[i].cstride; }
                if (i == 1 && net->fused_into_next[0] == 2) g.s2d_input = true;
                if (i == 0) {
                    if (L.in.c > 4) {  // generic first layer: quantise the image, then a normal convolution
                        QStep q;
                        q.layer = i; q.op = 7;
                        int64_t cs = ln_round_up(L.in.c, 32);
                        int b = alloc_buffer((int64_t)mb * L.in.h * L.in.w * cs);
                        if (b < 0) return LN_ERR_CUDA;
                        q.y = (uint8_t*)net->buffers[b].first; q.ys = cs; q.C = L.in.c; q.H = L.in.h; q.W = L.in.w; q.inv_sy = 1.0f / sx;
                        net->steps.push_back(q);
                        g.x = q.y; g.x_pixel_stride = cs;
                    } else {
                        if (head) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #0 cannot be a head convolution in the 8-bit plan");
                        st.op = 2;
                        st.inv_sy = 1.0f / sx;  // input quantiser
                        net->steps.push_back(st);
                        break;
                    }
                } else {
                    g.x = net->views[i - 1].ptr; g.x_pixel_stride = net->views[i - 1].cstride;
                }
                g.groups = L.groups;
                if (L.groups > 1) { g.cpad = (int)ln_round_up(L.in.c, 32); g.w_cpad = (int)L.wq->cpad; }  // grouped / depthwise: CUDA-core kernels
                if (L.groups == 1 && g.x_pixel_stride >= g.cpad && g.F <= 4096 && ln_conv_umma_supported(g.cpad, g.k, g.stride, g.stride, 1, 1, g.W, g.H)) {
                    st.op = 0;
                    st.umma.mb = st.mb;
                    rc = ln_conv_umma_plan_build(ctx, &st.umma, g);
                    if (rc) return rc;
                } else st.op = 1;
                if (st.op != 0 && net->fused_into_next[i] == 1) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer #%d: a fused shortcut needs the tensor-core convolution", i);
                net->steps.push_back(st);
                break;
            }
            case K_MAXPOOL: {
                st.op = 3;
                st.x = net->views[i - 1].ptr; st.xs = net->views[i - 1].cstride;
                st.pool_size = L.size; st.pool_pad = L.padding;
                // SPP cascade: a centred stride-1 max over s x s equals a centred max over (s - s' + 1) of an earlier
                // centred s' x s' max of the same tensor (taps outside the image are skipped = -inf padding), e.g. 9 = 5 o 5
                if (L.stride_x == 1 && L.stride_y == 1 && (L.size & 1) && L.padding == L.size - 1) {
                    int best = -1;
                    for (int j = 0; j < i; ++j) {
                        const NLayer& P = net->layers[j];
                        if (P.kind != K_MAXPOOL || P.stride_x != 1 || P.stride_y != 1 || !(P.size & 1) || P.padding != P.size - 1 || P.size >= L.size) continue;
                        if (j == 0 || root_of(j - 1) != root_of(i - 1)) continue;
                        if (best < 0 || P.size > net->layers[best].size) best = j;
                    }
                    if (best >= 0) {
                        st.x = net->views[best].ptr; st.xs = net->views[best].cstride;
                        st.pool_size = L.size - net->layers[best].size + 1;
                        st.pool_pad = st.pool_size - 1;
                    }
                }
                st.y = net->views[i].ptr; st.ys = net->views[i].cstride;
                st.C = L.in.c; st.H = L.in.h; st.W = L.in.w; st.OH = L.out.h; st.OW = L.out.w;
                net->steps.push_back(st);
                break;
            }
            case K_UPSAMPLE: {
                const bool copy = !L.up_reverse && L.up_scale == 1.0f;
                st.op = copy ? 4 : 9;
                st.x = net->views[i - 1].ptr; st.xs = net->views[i - 1].cstride;
                st.y = net->views[i].ptr; st.ys = net->views[i].cstride;
                st.C = L.in.c; st.H = L.in.h; st.W = L.in.w;
                st.inv_sy = (sx * L.up_scale) / sy;  // requantisation factor of the scaling / reverse form
                net->steps.push_back(st);
                break;
            }
            case K_ROUTE: {
                if (L.sources.size() >= 2) {
                    int off = 0;
                    for (int s : L.sources) {
                        const int r = root_of(s);
                        if (!(home_buf[r] == i && home_off[r] == off)) {  // not produced in place: copy
                            QStep c;
                            c.layer = i; c.op = 5;
                            c.x = net->views[s].ptr; c.xs = net->views[s].cstride;
                            c.y = net->views[i].ptr + off; c.ys = net->views[i].cstride;
                            c.C = net->layers[s].out.c; c.H = L.out.h; c.W = L.out.w;
                            net->steps.push_back(c);
                        }
                        off += net->layers[s].out.c;
                    }
                } else if (alias[i] < 0) {
                    const int chunk = net->layers[L.sources[0]].out.c / L.route_groups, start = chunk * L.route_group_id;
                    if (start % 16 != 0) {
                        QStep c;
                        c.layer = i; c.op = 5;
                        c.x = net->views[L.sources[0]].ptr + start; c.xs = net->views[L.sources[0]].cstride;
                        c.y = net->views[i].ptr; c.ys = net->views[i].cstride;
                        c.C = chunk; c.H = L.out.h; c.W = L.out.w;
                        net->steps.push_back(c);
                    }
                }
                break;
            }
            case K_SHORTCUT: {
                if (net->fused_into_next[i - 1] == 1) break;  // done in the epilogue of the convolution before it
                st.op = 6;
                const int s = L.sources[0];
                st.x = net->views[i - 1].ptr; st.xs = net->views[i - 1].cstride; st.sa = sx;
                st.x2 = net->views[s].ptr; st.xs2 = net->views[s].cstride; st.sb = net->scale[s + 1];
                const Shape4& ss = net->layers[s].out;
                if (ss.w != L.out.w || ss.h != L.out.h || ss.c != L.out.c) {
                    // a source of another shape is cropped / zero-padded flat per sample into a buffer of this layer's shape first
                    QStep f;
                    f.layer = i; f.op = 8;
                    const int64_t cs = ln_round_up(L.out.c, 32);
                    const int b = alloc_buffer((int64_t)mb * L.out.h * L.out.w * cs);
                    if (b < 0) return LN_ERR_CUDA;
                    f.x = st.x2; f.xs = st.xs2; f.sc = ss.c; f.sh = ss.h; f.sw = ss.w;
                    f.y = (uint8_t*)net->buffers[b].first; f.ys = cs;
                    f.C = L.out.c; f.H = L.out.h; f.W = L.out.w;
                    net->steps.push_back(f);
                    st.x2 = f.y; st.xs2 = cs;
                }
                st.y = net->views[i].ptr; st.ys = net->views[i].cstride; st.inv_sy = 1.0f / sy;
                st.C = L.out.c; st.H = L.out.h; st.W = L.out.w;
                net->steps.push_back(st);
                break;
            }
            case K_YOLO: break;
        }
    }
    net->plan_valid = true;
    net->plan_mb = mb;
    return LN_OK;
}

int run_plan(ln_net* net, const float* input_dev_f32) {
    ln_ctx* ctx = net->ctx;
    const int mb = net->plan_mb;
    const int kind = net->precision == LN_F8 ? LN_KIND_F8 : LN_KIND_I8;
    const int64_t in_image = (int64_t)net->channels * net->height * net->width;
    size_t ev_index = 0;
    if (net->profile) {
        const size_t need = net->steps.size() * (size_t)(net->batch / mb) + 1;
        while (net->prof_events.size() < need) {
            cudaEvent_t e;
            LN_CUDA(ctx, cudaEventCreate(&e));
            net->prof_events.push_back(e);
        }
        LN_CUDA(ctx, cudaEventRecord(net->prof_events[ev_index++], ctx->stream));
    }
    for (int b0 = 0; b0 < net->batch; b0 += mb) {
        for (auto& st : net->steps) {
            const NLayer& L = net->layers[st.layer];
            int rc = LN_OK;
            switch (st.op) {
                case 0: {
                    if (st.head) {
                        ln_conv_umma_plan plan = st.umma;
                        plan.p.out = (float*)st.geom.out + (int64_t)b0 * L.out.c * L.out.h * L.out.w;
                        rc = ln_conv_umma_launch(ctx, &plan);
                    } else rc = ln_conv_umma_launch(ctx, &st.umma);
                    break;
                }
                case 1: {
                    ln_conv_geom g = st.geom;
                    if (st.head) g.out = (float*)st.geom.out + (int64_t)b0 * L.out.c * L.out.h * L.out.w;
                    rc = ln_conv_simt_launch(ctx, g, nullptr, st.mb);
                    break;
                }
                case 2:
                    rc = ln_conv_stem_launch(ctx, kind, input_dev_f32 + b0 * in_image, st.inv_sy, mb, L.in.c, L.in.h, L.in.w, L.wq->w_oihw, st.mb, L.filters, L.size,
                                             L.stride_x, L.padding, L.out.h, L.out.w, L.act, st.geom.inv_sy, st.geom.out, st.geom.out_pixel_stride, net->fused_into_next[0] == 2 ? 1 : 0);
                    break;
                case 3: rc = ln_q_maxpool_launch(ctx, kind, st.x, st.xs, st.y, st.ys, mb, st.C, st.H, st.W, st.OH, st.OW, st.pool_size, L.stride_x, L.stride_y, st.pool_pad); break;
                case 4: rc = ln_q_upsample_launch(ctx, st.x, st.xs, st.y, st.ys, mb, st.C, st.H, st.W, L.up_stride); break;
                case 5: rc = ln_q_copy_launch(ctx, st.x, st.xs, st.y, st.ys, (int64_t)mb * st.H * st.W, st.C); break;
                case 6: rc = ln_q_shortcut_launch(ctx, kind, st.x, st.xs, st.sa, st.x2, st.xs2, st.sb, st.y, st.ys, (int64_t)mb * st.H * st.W, st.C, L.act, st.inv_sy); break;
                case 8: rc = ln_q_shortcut_fit_launch(ctx, st.x, st.xs, st.sc, st.sh, st.sw, st.y, st.ys, mb, st.C, st.H, st.W); break;
                case 9: rc = ln_q_upsample_requant_launch(ctx, kind, st.x, st.xs, st.y, st.ys, mb, st.C, st.H, st.W, L.up_stride, L.up_reverse ? 1 : 0, st.inv_sy); break;
                case 7: rc = ln_q_quantize_launch(ctx, kind, input_dev_f32 + b0 * in_image, st.y, mb, st.C, st.H, st.W, st.ys, st.inv_sy); break;
            }
            if (rc) return rc;
            if (net->profile) LN_CUDA(ctx, cudaEventRecord(net->prof_events[ev_index++], ctx->stream));
        }
    }
    if (net->profile) {
        LN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        net->prof_layer_ms.assign(net->layers.size(), 0.0f);
        for (int i = 0; i < 8; ++i) { net->prof_op_ms[i] = 0; net->prof_op_launches[i] = 0; }
        size_t e = 0;
        for (int b0 = 0; b0 < net->batch; b0 += mb)
            for (auto& st : net->steps) {
                float ms = 0;
                cudaEventElapsedTime(&ms, net->prof_events[e], net->prof_events[e + 1]);
                ++e;
                net->prof_layer_ms[st.layer] += ms;
                net->prof_op_ms[st.op] += ms;
                net->prof_op_launches[st.op] += 1;
            }
    }
    return LN_OK;
}

int forward_any(ln_net* net, const ln_tensor* input) {
    ln_ctx* ctx = net->ctx;
    if (!net->weights_loaded) return ln_fail(ctx, LN_ERR_ARG, "weights are not loaded");
    if (!input || input->dtype != LN_F32 || input->n != net->batch || input->c != net->channels || input->h != net->height || input->w != net->width)
        return ln_fail(ctx, LN_ERR_SHAPE, "input tensor must be f32 [%d,%d,%d,%d]", net->batch, net->channels, net->height, net->width);
    cudaSetDevice(ctx->device);
    LN_CUDA(ctx, cudaEventRecord(net->ev[0], ctx->stream));
    int rc;
    if (net->precision == LN_F32) rc = forward_f32(net, input, nullptr);
    else if (net->precision == LN_F16) rc = forward_f16(net, input);
    else {
        int mb = net->micro_batch > 0 && net->micro_batch < net->batch ? net->micro_batch : net->batch;
        if (net->batch % mb != 0) return ln_fail(ctx, LN_ERR_ARG, "micro batch %d does not divide batch %d", mb, net->batch);
        if (!net->plan_valid || net->plan_mb != mb) {
            rc = build_plan(net, mb);
            if (rc) { release_plan(net); return rc; }
            LN_CUDA(ctx, cudaEventRecord(net->ev[0], ctx->stream));
        }
        if (!net->use_graph || net->profile) rc = run_plan(net, (const float*)input->ptr);
        else {
            // launch-bound otherwise (about a thousand launches per batch): replay one captured graph
            ln_net::GraphSlot* slot = nullptr;
            for (auto& g : net->graphs)
                if (g.used && g.input == input->ptr && g.exact == ctx->exact_epilogue) slot = &g;
            if (slot && slot->exec) {
                LN_CUDA(ctx, cudaGraphLaunch(slot->exec, ctx->stream));
                ctx->launches += (int64_t)net->steps.size() * (net->batch / mb);
                rc = LN_OK;
            } else if (!slot) {
                // first sight of this key: an eager run (kernel attributes get set here), and the key is remembered
                slot = &net->graphs[0];
                for (auto& g : net->graphs)
                    if (g.used < slot->used) slot = &g;
                if (slot->exec) cudaGraphExecDestroy(slot->exec);
                *slot = ln_net::GraphSlot();
                slot->input = input->ptr;
                slot->exact = ctx->exact_epilogue;
                rc = run_plan(net, (const float*)input->ptr);
            } else {
                cudaGraph_t graph = nullptr;
                LN_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
                rc = run_plan(net, (const float*)input->ptr);
                cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
                if (rc == LN_OK && e != cudaSuccess) rc = ln_fail(ctx, LN_ERR_CUDA, "graph capture: %s", cudaGetErrorString(e));
                if (rc == LN_OK) {
                    e = cudaGraphInstantiate(&slot->exec, graph, 0);
                    if (e != cudaSuccess) { slot->exec = nullptr; rc = ln_fail(ctx, LN_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
                }
                if (graph) cudaGraphDestroy(graph);
                if (rc == LN_OK) LN_CUDA(ctx, cudaGraphLaunch(slot->exec, ctx->stream));
            }
            slot->used = ++net->graph_clock;
        }
        if (rc == LN_OK) rc = ln_check_status(ctx, "ln_net_forward");
    }
    if (rc) return rc;
    // anchor-free heads: the head layer's own forward, on the raw f32 tensor the convolution before it wrote: the output activation
    // (lib.rs:4884), then for the distribution heads the device box decode (lib.rs:4936)
    for (size_t k = 0; k < net->head_layers.size() && k < net->heads.size(); ++k) {
        const NLayer& L = net->layers[net->head_layers[k]];
        if (!L.modern) continue;
        if (net->modern_heads.size() != net->head_layers.size()) net->modern_heads.assign(net->head_layers.size(), nullptr);
        if (net->modern_heads[k]) { ln_tensor_release(net->modern_heads[k]); net->modern_heads[k] = nullptr; }
        ln_tensor* act = nullptr;
        rc = ln_modern_yolo_forward_f32(ctx, net->heads[k], L.classes, &act);
        if (rc) return rc;
        if (L.modern == 1) net->modern_heads[k] = act;
        else {
            ln_tensor* boxes = nullptr;
            rc = ln_modern_yolo_predecode_f32(ctx, act, L.classes, L.modern_coords, L.modern - 1, &boxes);
            ln_tensor_release(act);
            if (rc) return rc;
            net->modern_heads[k] = boxes;
        }
    }
    LN_CUDA(ctx, cudaEventRecord(net->ev[1], ctx->stream));
    return LN_OK;
}

int fill_heads(ln_net* net, std::vector<ln_yolo_head>& hs, const std::vector<ln_tensor*>* tensors = nullptr) {
    const std::vector<ln_tensor*>& heads = tensors ? *tensors : net->heads;
    if (heads.size() != net->head_layers.size()) return ln_fail(net->ctx, LN_ERR_ARG, "no head output: run a forward first");
    hs.resize(net->head_layers.size());
    for (size_t k = 0; k < hs.size(); ++k) {
        const NLayer& L = net->layers[net->head_layers[k]];
        ln_yolo_head& h = hs[k];
        memset(&h, 0, sizeof h);
        h.raw = heads[k];
        if (L.modern) {
            if (tensors || k >= net->modern_heads.size() || !net->modern_heads[k]) return ln_fail(net->ctx, LN_ERR_UNSUPPORTED, "anchor-free heads are not run through the host-input pipeline");
            h.raw = net->modern_heads[k];
            h.kind = L.modern == 1 ? 1 : 2;
        }
        h.classes = L.classes;
        h.n_anchor = (int)L.mask.size();
        for (size_t m = 0; m < L.mask.size(); ++m) { h.anchors[2 * m] = L.anchors[2 * L.mask[m]]; h.anchors[2 * m + 1] = L.anchors[2 * L.mask[m] + 1]; }
        h.scale_x_y = L.scale_x_y;
        h.new_coords = L.new_coords ? 1 : 0;
    }
    return LN_OK;
}

// Sizes of the two parts of the host-input pipeline.  A step costs about 1.5 ms + 0.17 ms per image and the upload 0.09 ms per image
// (YOLOv4-608 on a B200): a short first part gets its upload out of the way quickly and its layers cover the upload of the long
// second part, which then runs at nearly whole-batch efficiency.  A quarter / three quarters split minimises the sum.
int pipe_batch(const ln_net* net, int part) {
    int first = net->batch >= 16 ? net->batch / 4 : net->batch / 2;
    if (const char* e = getenv("LN_PIPE_FIRST")) {  // tuning aid: images in the first part
        const int v = atoi(e);
        if (v >= 1 && v < net->batch) first = v;
    }
    return part == 0 ? first : net->batch - first;
}

void release_pipe(ln_net* net) {
    for (auto& c : net->pipe) {
        if (c) ln_net_destroy(c);
        c = nullptr;
    }
    for (auto*& t : net->pipe_heads) { ln_tensor_release(t); t = nullptr; }
    net->pipe_heads.clear();
}

// Builds (once) the two part-batch networks of the host-input pipeline from this network's cfg, weights and scales.
int ensure_pipe(ln_net* net) {
    ln_ctx* ctx = net->ctx;
    if (net->pipe[0] && net->pipe[1]) return LN_OK;
    release_pipe(net);
    std::vector<float> blob;
    for (auto& L : net->layers) {
        if (L.kind != K_CONV) continue;
        blob.insert(blob.end(), L.biases.begin(), L.biases.end());
        if (L.bn) {
            blob.insert(blob.end(), L.scales.begin(), L.scales.end());
            blob.insert(blob.end(), L.mean.begin(), L.mean.end());
            blob.insert(blob.end(), L.var.begin(), L.var.end());
        }
        blob.insert(blob.end(), L.weights.begin(), L.weights.end());
    }
    for (int hl : net->head_layers) {
        const NLayer& L = net->layers[hl];
        ln_tensor* t = ln_tensor_new(ctx, LN_F32, net->batch, L.out.c, L.out.h, L.out.w);
        if (!t) { release_pipe(net); return LN_ERR_CUDA; }
        net->pipe_heads.push_back(t);
    }
    for (int h = 0; h < 2; ++h) {
        int rc = ln_net_create(ctx, net->cfg_text.c_str(), pipe_batch(net, h), net->precision, &net->pipe[h]);
        if (rc == LN_OK) {
            for (ln_tensor* t : net->pipe_heads) net->pipe[h]->ext_heads.push_back(ln_tensor_view_batch(t, h == 0 ? 0 : pipe_batch(net, 0), pipe_batch(net, h)));
            net->pipe[h]->host_pipeline = false;
            net->pipe[h]->fuse_shortcut = net->fuse_shortcut;
            net->pipe[h]->use_graph = net->use_graph;
            rc = ln_net_load_weights(net->pipe[h], blob.data(), (int64_t)blob.size());
        }
        if (rc == LN_OK) rc = ln_net_set_scales(net->pipe[h], net->scale.data(), (int)net->scale.size());
        if (rc) { release_pipe(net); return rc; }
    }
    if (!net->copy_stream) {
        LN_CUDA(ctx, cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking));
        for (auto& e : net->copy_ev) LN_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    return LN_OK;
}

int stage_input(ln_net* net, const float* host) {
    ln_ctx* ctx = net->ctx;
    cudaSetDevice(ctx->device);
    if (!net->input_dev) {
        net->input_dev = ln_tensor_new(ctx, LN_F32, net->batch, net->channels, net->height, net->width);
        if (!net->input_dev) return LN_ERR_CUDA;
    }
    LN_CUDA(ctx, cudaMemcpyAsync(net->input_dev->ptr, host, (size_t)net->input_dev->count() * 4, cudaMemcpyHostToDevice, ctx->stream));
    return LN_OK;
}

}  // namespace

extern "C" {

int32_t ln_net_create(ln_ctx* ctx, const char* cfg_text, int32_t batch, int32_t precision, ln_net** out) {
    if (!ctx || !cfg_text || !out) return ln_fail(ctx, LN_ERR_ARG, "ln_net_create: NULL argument");
    if (precision != LN_F32 && precision != LN_F16 && precision != LN_Q8 && precision != LN_F8)
        return ln_fail(ctx, LN_ERR_ARG, "ln_net_create: precision must be LN_F32, LN_F16, LN_Q8 or LN_F8");
    std::unique_ptr<ln_net> net(new ln_net());
    net->ctx = ctx;
    net->precision = precision;
    try {
        net->cfg_text = cfg_text;
        build_layers(net.get(), cfg_text, batch);
    } catch (const ParseError& e) {
        return ln_fail(ctx, LN_ERR_PARSE, "%s", e.msg.c_str());
    } catch (const std::exception& e) {
        return ln_fail(ctx, LN_ERR_PARSE, "%s", e.what());
    }
    cudaSetDevice(ctx->device);
    for (auto& e : net->ev)
        if (cudaEventCreate(&e) != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "cudaEventCreate failed");
    *out = net.release();
    return LN_OK;
}

int32_t ln_net_destroy(ln_net* net) {
    if (!net) return LN_OK;
    cudaSetDevice(net->ctx->device);
    cudaStreamSynchronize(net->ctx->stream);
    release_plan(net);
    release_outputs(net);
    release_heads(net);
    for (auto*& t : net->ext_heads) { ln_tensor_release(t); t = nullptr; }
    ln_tensor_release(net->input_dev);
    if (net->copy_stream) cudaStreamSynchronize(net->copy_stream);  // a submitted batch that was never collected
    for (int i = 0; i < 2; ++i)
        if (net->slot_staging[i]) ln_pool_free(net->ctx, net->slot_staging[i], net->slot_staging_bytes[i]);
    for (auto& t : net->slot_dev) if (t) ln_tensor_release(t);
    for (auto& e : net->slot_ev) if (e) cudaEventDestroy(e);
    release_pipe(net);
    if (net->copy_stream) cudaStreamDestroy(net->copy_stream);
    for (auto& e : net->copy_ev) if (e) cudaEventDestroy(e);
    for (auto& L : net->layers) {
        ln_tensor_release(L.w_f32);
        ln_tensor_release(L.b_f32);
        ln_conv_weights_release(L.wq);
    }
    for (auto& e : net->ev) if (e) cudaEventDestroy(e);
    for (auto& e : net->prof_events) cudaEventDestroy(e);
    delete net;
    return LN_OK;
}

int32_t ln_net_num_layers(const ln_net* net) { return net ? (int)net->layers.size() : 0; }

int32_t ln_net_layer_info(const ln_net* net, int32_t layer, int32_t info[20]) {
    if (!net || !info || layer < 0 || layer >= (int)net->layers.size()) return LN_ERR_ARG;
    const NLayer& L = net->layers[layer];
    int v[20] = {L.kind, L.in.w, L.in.h, L.in.c, L.in.b, L.out.w, L.out.h, L.out.c, L.out.b, L.filters, L.size, L.stride_x, L.stride_y, L.padding, L.bn ? 1 : 0, L.act,
                 L.groups, L.dilation, 0, 0};
    memcpy(info, v, sizeof v);
    return LN_OK;
}

int64_t ln_net_weight_count(const ln_net* net) {
    int64_t c = 0;
    if (net)
        for (auto& L : net->layers)
            if (L.kind == K_CONV) c += (int64_t)L.biases.size() * (L.bn ? 4 : 1) + (int64_t)L.weights.size();
    return c;
}

int32_t ln_net_load_weights(ln_net* net, const float* blob, int64_t count) {
    if (!net || !blob) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_load_weights: NULL argument");
    ln_ctx* ctx = net->ctx;
    if (count != ln_net_weight_count(net)) return ln_fail(ctx, LN_ERR_SHAPE, "weight blob has %lld values, the network needs %lld", (long long)count, (long long)ln_net_weight_count(net));
    cudaSetDevice(ctx->device);
    release_plan(net);
    release_pipe(net);
    const float* w = blob;
    for (auto& L : net->layers) {
        if (L.kind != K_CONV) continue;
        auto take = [&](std::vector<float>& v) { memcpy(v.data(), w, v.size() * 4); w += v.size(); };
        take(L.biases);
        if (L.bn) { take(L.scales); take(L.mean); take(L.var); }
        take(L.weights);
        // fold_convolutional_params_for_inference (runtime/weights_io.rs:32-92)
        std::vector<float> fw = L.weights, fb = L.biases;
        if (L.bn) {
            const size_t per = fw.size() / L.filters;
            for (int f = 0; f < L.filters; ++f) {
                const float scale = L.scales[f] / std::sqrt(L.var[f] + 1e-5f);
                const float shift = L.mean[f] * scale;
                fb[f] = fb[f] - shift;
                for (size_t k = 0; k < per; ++k) fw[f * per + k] = fw[f * per + k] * scale;
            }
        }
        ln_tensor_release(L.w_f32); L.w_f32 = nullptr;
        ln_tensor_release(L.b_f32); L.b_f32 = nullptr;
        ln_conv_weights_release(L.wq); L.wq = nullptr;
        const int64_t wshape[4] = {L.filters, L.in.c / L.groups, L.size, L.size}, bshape[4] = {1, L.filters, 1, 1};
        int rc = ln_tensor_upload_f32(ctx, wshape, fw.data(), &L.w_f32);
        if (rc == LN_OK) rc = ln_tensor_upload_f32(ctx, bshape, fb.data(), &L.b_f32);
        if (rc == LN_OK) rc = ln_sync(ctx);  // the host vectors die at the end of this scope
        if (rc == LN_OK && net->precision == LN_F16)
            rc = ln_conv_weights_f16(ctx, L.w_f32, L.filters, (int64_t)(L.in.c / L.groups) * L.size * L.size, &L.wq);
        else if (rc == LN_OK && net->precision != LN_F32) {
            rc = ln_conv_weights_q(ctx, L.w_f32, L.filters, L.in.c / L.groups, L.size, net->precision, &L.wq);  // [filters][C / groups][k][k]
        }
        if (rc) return rc;
    }
    net->weights_loaded = true;
    return LN_OK;
}

int32_t ln_net_load_weights_file(ln_net* net, const char* path) {
    if (!net || !path) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_load_weights_file: NULL argument");
    std::ifstream f(path, std::ios::binary);
    if (!f) return ln_fail(net->ctx, LN_ERR_ARG, "cannot open %s", path);
    // read_header (runtime/weights_io.rs:911-928)
    int32_t hdr[3];
    f.read((char*)hdr, 12);
    if (!f) return ln_fail(net->ctx, LN_ERR_PARSE, "%s: truncated header", path);
    if (hdr[0] * 10 + hdr[1] >= 2) { uint64_t seen; f.read((char*)&seen, 8); } else { uint32_t seen; f.read((char*)&seen, 4); }
    const int64_t n = ln_net_weight_count(net);
    std::vector<float> blob((size_t)n);
    f.read((char*)blob.data(), n * 4);
    if (f.gcount() != n * 4) return ln_fail(net->ctx, LN_ERR_PARSE, "%s: expected %lld weight values after the header, file has %lld", path, (long long)n, (long long)(f.gcount() / 4));
    return ln_net_load_weights(net, blob.data(), n);
}

int32_t ln_net_calibrate(ln_net* net, const float* input_host) {
    if (!net || !input_host) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_calibrate: NULL argument");
    ln_ctx* ctx = net->ctx;
    if (!net->weights_loaded) return ln_fail(ctx, LN_ERR_ARG, "weights are not loaded");
    int rc = stage_input(net, input_host);
    if (rc) return rc;
    const int T = (int)net->layers.size() + 1;
    unsigned* amax_dev = (unsigned*)ln_pool_alloc(ctx, (size_t)T * 4);
    if (!amax_dev) return LN_ERR_CUDA;
    cudaMemsetAsync(amax_dev, 0, (size_t)T * 4, ctx->stream);
    rc = forward_f32(net, net->input_dev, amax_dev);
    std::vector<float> amax((size_t)T, 0.0f);
    if (rc == LN_OK) {
        cudaError_t e = cudaMemcpyAsync(amax.data(), amax_dev, (size_t)T * 4, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = ln_fail(ctx, LN_ERR_CUDA, "calibration download: %s", cudaGetErrorString(e));
    }
    ln_pool_free(ctx, amax_dev, (size_t)T * 4);
    release_outputs(net);
    release_heads(net);
    if (rc) return rc;
    scales_from_amax(net, amax, net->precision == LN_F8 ? 448.0f : 127.0f);
    release_plan(net);
    return LN_OK;
}

int32_t ln_net_get_scales(const ln_net* net, float* scales, int32_t count) {
    if (!net || !scales || count != (int)net->layers.size() + 1 || !net->scales_set) return LN_ERR_ARG;
    memcpy(scales, net->scale.data(), (size_t)count * 4);
    return LN_OK;
}

int32_t ln_net_set_scales(ln_net* net, const float* scales, int32_t count) {
    if (!net || !scales) return LN_ERR_ARG;
    if (count != (int)net->layers.size() + 1) return ln_fail(net->ctx, LN_ERR_SHAPE, "expected %d scales, got %d", (int)net->layers.size() + 1, count);
    for (int i = 0; i < count; ++i)
        if (!(scales[i] > 0.0f)) return ln_fail(net->ctx, LN_ERR_ARG, "scale %d is not positive", i);
    net->scale.assign(scales, scales + count);
    net->scales_set = true;
    release_plan(net);
    release_pipe(net);
    return LN_OK;
}

int32_t ln_net_set_micro_batch(ln_net* net, int32_t micro_batch) {
    if (!net || micro_batch < 0) return LN_ERR_ARG;
    if (micro_batch > 0 && net->batch % micro_batch != 0) return ln_fail(net->ctx, LN_ERR_ARG, "micro batch %d does not divide batch %d", micro_batch, net->batch);
    net->micro_batch = micro_batch;
    return LN_OK;
}

int32_t ln_net_forward_device(ln_net* net, const ln_tensor* input) {
    if (!net) return LN_ERR_ARG;
    return forward_any(net, input);
}

int32_t ln_net_forward(ln_net* net, const float* input_host) {
    if (!net || !input_host) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_forward: NULL argument");
    int rc = stage_input(net, input_host);
    if (rc) return rc;
    return forward_any(net, net->input_dev);
}

int32_t ln_net_num_heads(const ln_net* net) { return net ? (int)net->head_layers.size() : 0; }

int32_t ln_net_head(ln_net* net, int32_t head_index, ln_tensor** out) {
    if (!net || !out) return LN_ERR_ARG;
    if (head_index < 0 || head_index >= (int)net->heads.size()) return ln_fail(net->ctx, LN_ERR_ARG, "head %d is not available (run a forward first)", head_index);
    ln_tensor* t = head_index < (int)net->modern_heads.size() && net->modern_heads[head_index] ? net->modern_heads[head_index] : net->heads[head_index];
    ln_tensor_retain(t);
    *out = t;
    return LN_OK;
}

int32_t ln_net_layer_output(ln_net* net, int32_t layer, ln_tensor** out) {
    if (!net || !out || layer < 0 || layer >= (int)net->layers.size()) return LN_ERR_ARG;
    ln_ctx* ctx = net->ctx;
    if (net->precision == LN_F32 || net->precision == LN_F16) {
        if ((int)net->out.size() <= layer || !net->out[layer]) return ln_fail(ctx, LN_ERR_ARG, "layer %d has no output (run a forward first)", layer);
        ln_tensor_retain(net->out[layer]);
        *out = net->out[layer];
        return LN_OK;
    }
    if (!net->plan_valid || net->plan_mb != net->batch) return ln_fail(ctx, LN_ERR_ARG, "8-bit layer outputs are kept for whole-batch forwards only (micro batch 0)");
    const NLayer& L = net->layers[layer];
    if (L.kind == K_YOLO || feeds_head(net, layer)) {
        int k = 0;
        for (size_t h = 0; h < net->head_layers.size(); ++h)
            if (net->head_layers[h] == layer || net->head_layers[h] == layer + 1) k = (int)h;
        ln_tensor_retain(net->heads[k]);
        *out = net->heads[k];
        return LN_OK;
    }
    if (net->fused_into_next[layer]) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "layer %d is fused into the layer after it and has no output of its own in the standard layout (ln_net_set_fusion(0) keeps it)", layer);
    const QView& v = net->views[layer];
    // a copy, so that the handle stays valid after the plan is rebuilt
    ln_tensor* t = ln_tensor_new(ctx, net->precision, net->batch, v.c, v.h, v.w);
    if (!t) return LN_ERR_CUDA;
    t->scale = net->scale[layer + 1];
    cudaMemsetAsync(t->ptr, 0, t->bytes, ctx->stream);
    int rc = ln_q_copy_launch(ctx, v.ptr, v.cstride, t->ptr, t->cstride, (int64_t)net->batch * v.h * v.w, v.c);
    if (rc) { ln_tensor_release(t); return rc; }
    *out = t;
    return LN_OK;
}

int32_t ln_net_detect_device(ln_net* net, const ln_tensor* input, const int32_t* image_w, const int32_t* image_h, const ln_detect_options* opts,
                             ln_detection* records_host, int32_t* counts_host) {
    if (!net || !image_w || !image_h || !opts || !records_host || !counts_host) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_detect: NULL argument");
    int rc = forward_any(net, input);
    if (rc) return rc;
    std::vector<ln_yolo_head> hs;
    rc = fill_heads(net, hs);
    if (rc) return rc;
    rc = ln_yolo_decode_nms(net->ctx, hs.data(), (int)hs.size(), net->width, net->height, image_w, image_h, opts, records_host, counts_host);
    if (rc) return rc;
    ln_ctx* ctx = net->ctx;
    LN_CUDA(ctx, cudaEventRecord(net->ev[2], ctx->stream));
    LN_CUDA(ctx, cudaEventSynchronize(net->ev[2]));
    cudaEventElapsedTime(&net->times_ms[0], net->ev[0], net->ev[1]);
    cudaEventElapsedTime(&net->times_ms[1], net->ev[1], net->ev[2]);
    return LN_OK;
}

int32_t ln_net_detect(ln_net* net, const float* input_host, const int32_t* image_w, const int32_t* image_h, const ln_detect_options* opts,
                      ln_detection* records_host, int32_t* counts_host) {
    if (!net || !input_host) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_detect: NULL argument");
    ln_ctx* ctx = net->ctx;
    bool any_modern = false;
    for (int hl : net->head_layers) any_modern = any_modern || net->layers[hl].modern != 0;
    if (!any_modern && (net->precision == LN_Q8 || net->precision == LN_F8) && net->host_pipeline && net->batch >= 8 && net->batch % 2 == 0 && net->weights_loaded && net->scales_set &&
        image_w && image_h && opts && records_host && counts_host && opts->max_per_image >= 1) {
        int rc = ensure_pipe(net);
        if (rc) return rc;
        cudaSetDevice(ctx->device);
        const size_t in_image = (size_t)net->channels * net->height * net->width;
        int start[2] = {0, pipe_batch(net, 0)};
        for (int h = 0; h < 2; ++h) {
            ln_net* c = net->pipe[h];
            if (!c->input_dev) {
                c->input_dev = ln_tensor_new(ctx, LN_F32, c->batch, net->channels, net->height, net->width);
                if (!c->input_dev) return LN_ERR_CUDA;
            }
            // every earlier call has synchronised the compute stream before it returned: nothing still reads these buffers
            LN_CUDA(ctx, cudaMemcpyAsync(c->input_dev->ptr, input_host + (size_t)start[h] * in_image, (size_t)c->batch * in_image * 4, cudaMemcpyHostToDevice,
                                         net->copy_stream));
            LN_CUDA(ctx, cudaEventRecord(net->copy_ev[h], net->copy_stream));
        }
        // both parts' layers (the second waits for its upload), each writing its image range of the shared heads, then one
        // decode + NMS over the whole batch
        for (int h = 0; h < 2; ++h) {
            ln_net* c = net->pipe[h];
            LN_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, net->copy_ev[h], 0));
            rc = forward_any(c, c->input_dev);
            if (rc) return rc;
        }
        std::vector<ln_yolo_head> hs;
        rc = fill_heads(net, hs, &net->pipe_heads);
        if (rc) return rc;
        rc = ln_yolo_decode_nms(ctx, hs.data(), (int)hs.size(), net->width, net->height, image_w, image_h, opts, records_host, counts_host);
        if (rc) return rc;
        LN_CUDA(ctx, cudaEventRecord(net->ev[2], ctx->stream));
        LN_CUDA(ctx, cudaEventSynchronize(net->ev[2]));
        float part[2] = {0.0f, 0.0f}, nms = 0.0f;
        for (int h = 0; h < 2; ++h) cudaEventElapsedTime(&part[h], net->pipe[h]->ev[0], net->pipe[h]->ev[1]);
        cudaEventElapsedTime(&nms, net->pipe[1]->ev[1], net->ev[2]);
        net->times_ms[0] = part[0] + part[1];
        net->times_ms[1] = nms;
        return LN_OK;
    }
    int rc = stage_input(net, input_host);
    if (rc) return rc;
    return ln_net_detect_device(net, net->input_dev, image_w, image_h, opts, records_host, counts_host);
}

// Common part of the two submit calls: the copy stream, the slot of the next batch and its device tensor.
static int submit_slot(ln_net* net, const char* who, int* slot_out) {
    ln_ctx* ctx = net->ctx;
    if (net->submitted - net->collected >= 2) return ln_fail(ctx, LN_ERR_ARG, "%s: two batches are in flight already; collect one first", who);
    cudaSetDevice(ctx->device);
    if (!net->copy_stream) {
        LN_CUDA(ctx, cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking));
        for (auto& e : net->copy_ev) LN_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    const int slot = (int)(net->submitted & 1);
    if (!net->slot_dev[slot]) {
        net->slot_dev[slot] = ln_tensor_new(ctx, LN_F32, net->batch, net->channels, net->height, net->width);
        if (!net->slot_dev[slot]) return LN_ERR_CUDA;
        LN_CUDA(ctx, cudaEventCreateWithFlags(&net->slot_ev[slot], cudaEventDisableTiming));
    }
    *slot_out = slot;
    return LN_OK;
}

int32_t ln_net_submit(ln_net* net, const float* input_host) {
    if (!net || !input_host) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_submit: NULL argument");
    ln_ctx* ctx = net->ctx;
    int slot = 0;
    int rc = submit_slot(net, "ln_net_submit", &slot);
    if (rc) return rc;
    // the slot's previous batch was collected (its forward has been synchronised), so nothing reads the buffer any more
    LN_CUDA(ctx, cudaMemcpyAsync(net->slot_dev[slot]->ptr, input_host, (size_t)net->slot_dev[slot]->count() * 4, cudaMemcpyHostToDevice, net->copy_stream));
    LN_CUDA(ctx, cudaEventRecord(net->slot_ev[slot], net->copy_stream));
    net->submitted++;
    return LN_OK;
}

int32_t ln_net_submit_u8(ln_net* net, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths, const int32_t* heights,
                         int32_t mode) {
    if (!net || !pixels_host || !offsets || !widths || !heights) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_submit_u8: NULL argument");
    ln_ctx* ctx = net->ctx;
    if (net->channels != 3) return ln_fail(ctx, LN_ERR_SHAPE, "ln_net_submit_u8: the network takes %d channels, RGB images have 3", net->channels);
    int slot = 0;
    int rc = submit_slot(net, "ln_net_submit_u8", &slot);
    if (rc) return rc;
    // The staging block comes from the ctx pool, whose blocks may have been handed back in ctx-stream order: whatever that stream
    // holds right now goes first (nothing, in a submit / collect loop: every collect ends synchronised).
    LN_CUDA(ctx, cudaEventRecord(net->slot_ev[slot], ctx->stream));
    LN_CUDA(ctx, cudaStreamWaitEvent(net->copy_stream, net->slot_ev[slot], 0));
    // upload and resize both run on the copy stream, under the layers of the batch submitted before
    rc = ln_image_preprocess_enqueue(ctx, net->copy_stream, pixels_host, offsets, widths, heights, net->batch, mode, net->width, net->height,
                                     (float*)net->slot_dev[slot]->ptr, &net->slot_staging[slot], &net->slot_staging_bytes[slot]);
    if (rc) {
        if (net->slot_staging[slot]) {  // (something may have been enqueued before the failure)
            cudaStreamSynchronize(net->copy_stream);
            ln_pool_free(ctx, net->slot_staging[slot], net->slot_staging_bytes[slot]);
            net->slot_staging[slot] = nullptr;
        }
        return rc;
    }
    LN_CUDA(ctx, cudaEventRecord(net->slot_ev[slot], net->copy_stream));
    net->submitted++;
    return LN_OK;
}

int32_t ln_net_collect(ln_net* net, const int32_t* image_w, const int32_t* image_h, const ln_detect_options* opts, ln_detection* records_host,
                       int32_t* counts_host) {
    if (!net) return ln_fail(nullptr, LN_ERR_ARG, "ln_net_collect: NULL argument");
    ln_ctx* ctx = net->ctx;
    if (net->submitted == net->collected) return ln_fail(ctx, LN_ERR_ARG, "ln_net_collect: no batch has been submitted");
    cudaSetDevice(ctx->device);
    const int slot = (int)(net->collected & 1);
    net->collected++;  // (the slot is free again whatever happens below: every path out of ln_net_detect_device has synchronised or failed)
    int rc = LN_OK;
    cudaError_t e = cudaStreamWaitEvent(ctx->stream, net->slot_ev[slot], 0);
    if (e != cudaSuccess) rc = ln_fail(ctx, LN_ERR_CUDA, "ln_net_collect: %s", cudaGetErrorString(e));
    else rc = ln_net_detect_device(net, net->slot_dev[slot], image_w, image_h, opts, records_host, counts_host);
    if (net->slot_staging[slot]) {
        if (rc) cudaStreamSynchronize(net->copy_stream);  // an early failure may have left the resize in flight
        ln_pool_free(ctx, net->slot_staging[slot], net->slot_staging_bytes[slot]);
        net->slot_staging[slot] = nullptr;
    }
    return rc;
}

int32_t ln_net_detect_u8(ln_net* net, const uint8_t* pixels_host, const int64_t* offsets, const int32_t* widths, const int32_t* heights,
                         int32_t mode, const ln_detect_options* opts, ln_detection* records_host, int32_t* counts_host) {
    if (!net || !pixels_host || !offsets || !widths || !heights) return ln_fail(net ? net->ctx : nullptr, LN_ERR_ARG, "ln_net_detect_u8: NULL argument");
    ln_ctx* ctx = net->ctx;
    if (net->channels != 3) return ln_fail(ctx, LN_ERR_SHAPE, "ln_net_detect_u8: the network takes %d channels, RGB images have 3", net->channels);
    cudaSetDevice(ctx->device);
    if (!net->input_dev) {
        net->input_dev = ln_tensor_new(ctx, LN_F32, net->batch, net->channels, net->height, net->width);
        if (!net->input_dev) return LN_ERR_CUDA;
    }
    // (the two-part pipeline of ln_net_detect does not pay here: the 8-bit upload is a quarter of the f32 one, and two part-batch
    // networks with two decode + NMS calls cost more than overlapping it saves -- measured 4212 against 4630 images/s with halves)
    int rc = ln_image_preprocess_into(ctx, pixels_host, offsets, widths, heights, net->batch, mode, net->width, net->height, (float*)net->input_dev->ptr);
    if (rc) return rc;
    return ln_net_detect_device(net, net->input_dev, widths, heights, opts, records_host, counts_host);
}

int32_t ln_net_set_host_pipeline(ln_net* net, int32_t on) {
    if (!net) return LN_ERR_ARG;
    net->host_pipeline = on != 0;
    if (!net->host_pipeline) release_pipe(net);
    return LN_OK;
}

int32_t ln_net_set_cuda_graph(ln_net* net, int32_t on) {
    if (!net) return LN_ERR_ARG;
    net->use_graph = on != 0;
    if (!net->use_graph) release_graph(net);
    for (ln_net* c : net->pipe)  // the part networks of the host-input pipeline follow their owner
        if (c) ln_net_set_cuda_graph(c, on);
    return LN_OK;
}

int32_t ln_net_set_fusion(ln_net* net, int32_t on) {
    if (!net) return LN_ERR_ARG;
    net->fuse_shortcut = on != 0;
    release_plan(net);
    release_pipe(net);  // the part networks of the host-input pipeline are rebuilt with the new setting on the next host-input call
    return LN_OK;
}

int32_t ln_net_set_profile(ln_net* net, int32_t on) {
    if (!net) return LN_ERR_ARG;
    net->profile = on != 0;
    return LN_OK;
}

int32_t ln_net_profile(const ln_net* net, float* per_layer_ms, int32_t num_layers, float per_op_ms[8], int32_t per_op_launches[8]) {
    if (!net || !per_layer_ms || !per_op_ms || !per_op_launches) return LN_ERR_ARG;
    if (num_layers != (int)net->layers.size() || net->prof_layer_ms.size() != net->layers.size())
        return ln_fail(net->ctx, LN_ERR_ARG, "no profile: enable profiling and run an 8-bit forward first");
    memcpy(per_layer_ms, net->prof_layer_ms.data(), (size_t)num_layers * 4);
    memcpy(per_op_ms, net->prof_op_ms, sizeof net->prof_op_ms);
    memcpy(per_op_launches, net->prof_op_launches, sizeof net->prof_op_launches);
    return LN_OK;
}

int32_t ln_net_last_times(const ln_net* net, float times_ms[2]) {
    if (!net || !times_ms) return LN_ERR_ARG;
    times_ms[0] = net->times_ms[0];
    times_ms[1] = net->times_ms[1];
    return LN_OK;
}

}  // extern "C"
