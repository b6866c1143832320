// lightnet_oracle.cpp -- CPU restatement of the lightnet detector-inference path.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It is the checker the parity
// tests, the smoke entry and the bench's cpu_baseline leg compare the CUDA path
// against.  Nothing in the shipped library links, imports or executes it.
//
// Parity status:
//   * f32 path (cfg parse, shape rules, conv, BN, activations, maxpool, route,
//     shortcut, upsample, yolo decode, NMS, FP8 E4M3 codec): PINNED against the
//     known-answer tests the reference carries for this path (see
//     tests/test_oracle_kats.py, which cites each one).
//   * int8 quantiser / int8 network: the reference has no int8 path, so the
//     quantisation scheme itself is "parity unpinned"; it is defined here and the
//     CUDA path is held bit-exact to this definition.
//
// Every function cites the reference file:line (paths inside the lightnet
// project) whose behaviour it restates.  Plain scalar C++17, built with
// `g++ -O2 -ffp-contract=off` (no fast-math) so that no multiply-add is contracted:
// the reference is Rust, which never contracts.
//
// The optional OpenMP parallelism is over (image, filter) / (image) only; the
// accumulation order of every single output value is unchanged, so results are
// identical for any thread count.

#include <algorithm>
#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <numeric>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace orc {

// ---------------------------------------------------------------------------
// Model vocabulary
// ---------------------------------------------------------------------------

enum Act { ACT_LINEAR = 0, ACT_LOGISTIC = 1, ACT_LEAKY = 2, ACT_MISH = 3, ACT_SWISH = 4, ACT_RELU = 5 };
enum Kind { K_CONV = 0, K_MAXPOOL = 1, K_ROUTE = 2, K_SHORTCUT = 3, K_UPSAMPLE = 4, K_YOLO = 5 };

// lightnet-model/src/model.rs:19 TensorShape{width,height,channels,batch}
struct Shape {
    int w = 0, h = 0, c = 0, b = 0;
    size_t count() const { return (size_t)w * h * c * b; }
};

// lightnet-model/src/model.rs:48,98  planar NCHW f32, offset = ((b*C+c)*H+y)*W+x
struct Tensor {
    Shape s;
    std::vector<float> d;
    Tensor() {}
    explicit Tensor(Shape sh) : s(sh), d(sh.count(), 0.0f) {}
    size_t off(int b, int c, int y, int x) const { return (((size_t)b * s.c + c) * s.h + y) * s.w + x; }
    float get(int b, int c, int y, int x) const { return d[off(b, c, y, x)]; }
    void set(int b, int c, int y, int x, float v) { d[off(b, c, y, x)] = v; }
};

struct TensorI8 {
    Shape s;
    std::vector<int8_t> d;  // NCHW
    TensorI8() {}
    explicit TensorI8(Shape sh) : s(sh), d(sh.count(), 0) {}
    size_t off(int b, int c, int y, int x) const { return (((size_t)b * s.c + c) * s.h + y) * s.w + x; }
};

struct Layer {
    Kind kind = K_CONV;
    Shape in, out;
    // convolutional (model.rs:4088-4144)
    int filters = 1, size = 1, stride_x = 1, stride_y = 1, dilation = 1, padding = 0, groups = 1;
    bool bn = false;
    Act act = ACT_LOGISTIC;
    // route / shortcut: absolute source indices
    std::vector<int> sources;
    int route_groups = 1, route_group_id = 0;
    // upsample
    int up_stride = 2;
    float up_scale = 1.0f;
    bool up_reverse = false;
    // yolo
    int classes = 20, num = 1;
    std::vector<int> mask;
    std::vector<float> anchors;
    float scale_x_y = 1.0f;
    bool new_coords = false;
    // parameters (lightnet-layers/src/params.rs:7-26)
    std::vector<float> biases, scales, mean, var, weights;
    // int8 model
    std::vector<int8_t> wq;      // [filters][C/g][k][k]
    std::vector<float> wscale;   // per filter
    std::vector<float> fbias;    // folded bias
    // FP8 E4M3 model: per-filter scale max|w|/448, codes
    std::vector<uint8_t> w8;
    std::vector<float> w8scale;
};

struct Net {
    int width = 0, height = 0, channels = 0, batch = 1;
    std::vector<Layer> layers;
    // per-run state
    std::vector<Tensor> out_f32;
    std::vector<TensorI8> out_q8;
    std::vector<Tensor> head_q8;          // f32 heads of the int8 run, indexed by layer
    std::vector<std::vector<uint8_t>> out_f8;  // E4M3 codes, NCHW, per layer (FP8 run)
    std::vector<Tensor> head_f8;
    std::vector<float> amax;              // [0] = input, [1+i] = layer i output (f32 run)
    std::vector<float> scale;             // same indexing; per-tensor activation scale
    std::string error;
};

// ---------------------------------------------------------------------------
// cfg parsing: lightnet-model/src/cfg.rs:109-171 (sections, comments, lower-case
// keys, last value wins) and :183-195 (lists split on ',' or whitespace).
// ---------------------------------------------------------------------------

struct Section {
    std::string name;
    int line = 0;
    std::map<std::string, std::string> kv;
    bool has(const std::string& k) const { return kv.count(k) != 0; }
    std::string str(const std::string& k, const std::string& d) const {
        auto it = kv.find(k);
        return it == kv.end() ? d : it->second;
    }
    long long i64(const std::string& k, long long d) const {
        auto it = kv.find(k);
        if (it == kv.end()) return d;
        try {
            size_t pos = 0;
            long long v = std::stoll(it->second, &pos);
            if (pos != it->second.size()) throw std::invalid_argument("x");
            return v;
        } catch (...) { throw std::runtime_error("invalid integer for key " + k + " in [" + name + "]"); }
    }
    int usz(const std::string& k, int d) const {
        long long v = i64(k, d);
        if (v < 0) throw std::runtime_error("negative value for key " + k + " in [" + name + "]");
        return (int)v;
    }
    float f32(const std::string& k, float d) const {
        auto it = kv.find(k);
        if (it == kv.end()) return d;
        try { return std::stof(it->second); } catch (...) { throw std::runtime_error("invalid float for key " + k); }
    }
    bool flag(const std::string& k, bool d) const { return i64(k, d ? 1 : 0) != 0; }  // cfg.rs:78
};

static std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace((unsigned char)s[a])) ++a;
    while (b > a && std::isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
}
static std::string lower(std::string s) {
    for (auto& ch : s) ch = (char)std::tolower((unsigned char)ch);
    return s;
}

static std::vector<Section> parse_cfg(const std::string& text) {
    std::vector<Section> secs;
    std::istringstream in(text);
    std::string raw;
    int ln = 0;
    bool have = false;
    while (std::getline(in, raw)) {
        ++ln;
        std::string line = raw;
        size_t p = line.find('#');
        if (p != std::string::npos) line = line.substr(0, p);
        p = line.find(';');
        if (p != std::string::npos) line = line.substr(0, p);
        line = trim(line);
        if (line.empty()) continue;
        if (line.front() == '[' && line.back() == ']') {
            Section s;
            s.name = lower(trim(line.substr(1, line.size() - 2)));
            s.line = ln;
            secs.push_back(s);
            have = true;
            continue;
        }
        size_t eq = line.find('=');
        if (eq == std::string::npos) throw std::runtime_error("invalid config line " + std::to_string(ln) + ": expected key=value");
        if (!have) throw std::runtime_error("key/value before any section at line " + std::to_string(ln));
        secs.back().kv[lower(trim(line.substr(0, eq)))] = trim(line.substr(eq + 1));
    }
    if (secs.empty()) throw std::runtime_error("no Darknet sections found");
    return secs;
}

template <class T>
static std::vector<T> parse_list(const Section& s, const std::string& key) {
    std::vector<T> out;
    auto it = s.kv.find(key);
    if (it == s.kv.end()) return out;
    std::string item;
    auto flush = [&]() {
        if (item.empty()) return;
        try {
            if (std::is_floating_point<T>::value) out.push_back((T)std::stof(item));
            else out.push_back((T)std::stoll(item));
        } catch (...) { throw std::runtime_error("failed to parse list item \"" + item + "\" for key " + key); }
        item.clear();
    };
    for (char ch : it->second) {
        if (ch == ',' || std::isspace((unsigned char)ch)) flush();
        else item.push_back(ch);
    }
    flush();
    return out;
}

// model.rs:377 Activation::parse (subset reachable from the detector cfgs)
static Act parse_act(const std::string& s) {
    std::string a = lower(s);
    if (a == "linear") return ACT_LINEAR;
    if (a == "logistic") return ACT_LOGISTIC;
    if (a == "leaky") return ACT_LEAKY;
    if (a == "mish") return ACT_MISH;
    if (a == "swish") return ACT_SWISH;
    if (a == "relu") return ACT_RELU;
    throw std::runtime_error("activation \"" + s + "\" is outside the oracle's scope");
}

// model.rs:6472 conv_dim, model.rs:8854 pool_dim
static int conv_dim(int in, int pad, int size, int stride) {
    int v = in + 2 * pad - size;
    if (v < 0) v = 0;
    return v / std::max(stride, 1) + 1;
}
static int pool_dim(int in, int pad, int size, int stride) {
    int v = in + pad - size;
    if (v < 0) v = 0;
    return v / std::max(stride, 1) + 1;
}

// model.rs:6208 resolve_relative_layer
static int resolve_rel(int layer_index, long long raw) {
    long long a = raw < 0 ? layer_index + raw : raw;
    if (a < 0 || a >= layer_index) throw std::runtime_error("invalid route reference at layer " + std::to_string(layer_index));
    return (int)a;
}

// model.rs:3079 Network::from_config, restricted to the six layer kinds on the path.
static std::unique_ptr<Net> build_net(const std::string& cfg, int batch_override) {
    auto secs = parse_cfg(cfg);
    auto net = std::make_unique<Net>();
    const Section& n = secs[0];
    if (n.name != "net" && n.name != "network") throw std::runtime_error("first section must be [net]");
    net->width = n.usz("width", 0);
    net->height = n.usz("height", 0);
    net->channels = n.usz("channels", 0);
    // model.rs:247-249: batch = batch / subdivisions * time_steps
    int subdiv = std::max(n.usz("subdivisions", 1), 1);
    int ts = std::max(n.usz("time_steps", 1), 1);
    net->batch = n.usz("batch", 1) / subdiv * ts;
    if (batch_override > 0) net->batch = batch_override;  // model.rs:3256 with_batch
    Shape cur;
    cur.w = net->width; cur.h = net->height; cur.c = net->channels; cur.b = net->batch;
    for (size_t si = 1; si < secs.size(); ++si) {
        const Section& s = secs[si];
        int li = (int)net->layers.size();
        Layer L;
        L.in = cur;
        if (s.name == "conv" || s.name == "convolutional") {
            L.kind = K_CONV;
            int stride = s.usz("stride", 1);
            L.size = s.usz("size", 1);
            bool pad = s.flag("pad", false);
            L.padding = pad ? L.size / 2 : s.usz("padding", 0);
            L.filters = s.usz("filters", 1);
            L.groups = s.usz("groups", 1);
            L.stride_x = s.usz("stride_x", stride);
            L.stride_y = s.usz("stride_y", stride);
            L.dilation = s.usz("dilation", 1);
            L.bn = s.i64("batch_normalize", 0) != 0;
            L.act = parse_act(s.str("activation", "logistic"));
            L.out.w = conv_dim(cur.w, L.padding, L.size, L.stride_x);
            L.out.h = conv_dim(cur.h, L.padding, L.size, L.stride_y);
            L.out.c = L.filters;
            L.out.b = cur.b;
            int g = std::max(L.groups, 1);
            if (L.filters % g || cur.c % g) throw std::runtime_error("conv groups do not divide channels");
            size_t wn = (size_t)L.filters * (cur.c / g) * L.size * L.size;
            L.biases.assign(L.filters, 0.0f);
            L.weights.assign(wn, 0.0f);
            if (L.bn) {
                L.scales.assign(L.filters, 1.0f);
                L.mean.assign(L.filters, 0.0f);
                L.var.assign(L.filters, 1.0f);
            }
        } else if (s.name == "max" || s.name == "maxpool") {
            L.kind = K_MAXPOOL;
            int stride = s.usz("stride", 1);
            L.size = s.usz("size", stride);
            L.stride_x = s.usz("stride_x", stride);
            L.stride_y = s.usz("stride_y", stride);
            L.padding = s.usz("padding", L.size > 0 ? L.size - 1 : 0);
            if (s.flag("maxpool_depth", false)) throw std::runtime_error("maxpool_depth is outside the oracle's scope");
            L.out.w = pool_dim(cur.w, L.padding, L.size, L.stride_x);
            L.out.h = pool_dim(cur.h, L.padding, L.size, L.stride_y);
            L.out.c = cur.c;
            L.out.b = cur.b;
        } else if (s.name == "route") {
            L.kind = K_ROUTE;
            auto raw = parse_list<long long>(s, "layers");
            if (raw.empty()) throw std::runtime_error("route must list at least one source layer");
            L.route_groups = s.usz("groups", 1);
            L.route_group_id = s.usz("group_id", 0);
            int ch = 0;
            Shape first;
            for (size_t k = 0; k < raw.size(); ++k) {
                int src = resolve_rel(li, raw[k]);
                L.sources.push_back(src);
                const Shape& sh = net->layers[src].out;
                if (k == 0) first = sh;
                else if (sh.w != first.w || sh.h != first.h) throw std::runtime_error("route mixes incompatible spatial shapes");
                ch += sh.c;
            }
            // model.rs:6138 infer_route_shape
            L.out.w = first.w; L.out.h = first.h; L.out.c = ch / std::max(L.route_groups, 1); L.out.b = cur.b;
        } else if (s.name == "shortcut") {
            L.kind = K_SHORTCUT;
            auto raw = parse_list<long long>(s, "from");
            for (auto r : raw) L.sources.push_back(resolve_rel(li, r));
            L.act = parse_act(s.str("activation", "linear"));
            L.out = cur;
        } else if (s.name == "upsample") {
            L.kind = K_UPSAMPLE;
            long long st = s.i64("stride", 2);
            L.up_reverse = st < 0;
            L.up_stride = (int)std::llabs(st);
            if (L.up_stride == 0) throw std::runtime_error("upsample cannot use stride=0");
            L.up_scale = s.f32("scale", 1.0f);
            L.out = cur;
            if (L.up_reverse) { L.out.w = cur.w / L.up_stride; L.out.h = cur.h / L.up_stride; }
            else { L.out.w = cur.w * L.up_stride; L.out.h = cur.h * L.up_stride; }
        } else if (s.name == "yolo" || s.name == "gaussian_yolo") {
            // model.rs:4271-4344 and :4513-4543: at inference [gaussian_yolo] is the same identity layer with the same spec, decoded
            // by the same function (detect.rs:78, :135); its num is max(len(mask), num)
            L.kind = K_YOLO;
            L.mask = parse_list<int>(s, "mask");
            L.num = s.usz("num", L.mask.empty() ? 1 : (int)L.mask.size());
            if (s.name == "gaussian_yolo" && L.num < (int)L.mask.size()) L.num = (int)L.mask.size();
            if (L.mask.empty()) for (int k = 0; k < L.num; ++k) L.mask.push_back(k);
            L.classes = s.usz("classes", 20);
            L.anchors = parse_list<float>(s, "anchors");
            L.scale_x_y = s.f32("scale_x_y", 1.0f);
            L.new_coords = s.i64("new_coords", 0) != 0;
            L.out = cur;
        } else {
            throw std::runtime_error("layer [" + s.name + "] is outside the oracle's scope");
        }
        cur = L.out;
        net->layers.push_back(std::move(L));
    }
    return net;
}

// ---------------------------------------------------------------------------
// f32 layer math
// ---------------------------------------------------------------------------

static const float BN_EPS = 1e-5f;  // lightnet-layers/src/params.rs:4

// runtime/layer_ops.rs:1682-1695 normalize_value
static inline float normalize_value(float v, int idx, const Layer& L) {
    if (L.bn) {
        float normalized = (v - L.mean[idx]) / std::sqrt(L.var[idx] + BN_EPS);
        return normalized * L.scales[idx] + L.biases[idx];
    }
    return v + L.biases[idx];
}

// runtime/layer_ops.rs:1697-1738 activate (libm f32)
static inline float activate(Act a, float v) {
    switch (a) {
        case ACT_LINEAR: return v;
        case ACT_LOGISTIC: return 1.0f / (1.0f + std::exp(-v));
        case ACT_RELU: return std::max(v, 0.0f);
        case ACT_LEAKY: return v > 0.0f ? v : 0.1f * v;
        case ACT_MISH: return v * std::tanh(std::log(1.0f + std::exp(v)));
        case ACT_SWISH: return v / (1.0f + std::exp(-v));
    }
    return v;
}

// runtime/forward_layers.rs:610-699 forward_convolutional_with_cache.
// `folded` = use BN-folded weights/bias (runtime/weights_io.rs:32-92) instead of
// the unfolded normalize_value; the GPU path of the reference folds, the CPU path
// does not.
static void conv_f32(const Layer& L, const Tensor& x, Tensor& y, bool folded, const std::vector<float>* fw,
                     const std::vector<float>* fb) {
    const int g = std::max(L.groups, 1);
    const int fpg = L.filters / g, cpg = x.s.c / g;
    const float* W = folded ? fw->data() : L.weights.data();
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < x.s.b; ++b) {
        for (int f = 0; f < L.filters; ++f) {
            const int group = f / std::max(fpg, 1);
            for (int oy = 0; oy < y.s.h; ++oy) {
                for (int ox = 0; ox < y.s.w; ++ox) {
                    float acc = 0.0f;
                    for (int ic = 0; ic < cpg; ++ic) {
                        for (int ky = 0; ky < L.size; ++ky) {
                            for (int kx = 0; kx < L.size; ++kx) {
                                int sy = oy * L.stride_y + ky * L.dilation - L.padding;
                                int sx = ox * L.stride_x + kx * L.dilation - L.padding;
                                if (sy < 0 || sy >= x.s.h || sx < 0 || sx >= x.s.w) continue;
                                int ch = group * cpg + ic;
                                float iv = x.d[x.off(b, ch, sy, sx)];
                                size_t wi = (((size_t)f * cpg + ic) * L.size + ky) * L.size + kx;
                                acc += iv * W[wi];
                            }
                        }
                    }
                    float biased = folded ? acc + (*fb)[f] : normalize_value(acc, f, L);
                    y.d[y.off(b, f, oy, ox)] = activate(L.act, biased);
                }
            }
        }
    }
}

// runtime/weights_io.rs:32-92 fold_convolutional_params_for_inference
static void fold_bn(const Layer& L, int in_c, std::vector<float>& fw, std::vector<float>& fb) {
    fw = L.weights;
    fb = L.biases;
    if (!L.bn) return;
    const int g = std::max(L.groups, 1);
    size_t per = (size_t)(in_c / g) * L.size * L.size;
    for (int f = 0; f < L.filters; ++f) {
        float scale = L.scales[f] / std::sqrt(L.var[f] + BN_EPS);
        fb[f] -= L.mean[f] * scale;
        for (size_t k = 0; k < per; ++k) fw[f * per + k] *= scale;
    }
}

// runtime/layer_ops.rs:1740-1799 forward_maxpool (average=false)
static void maxpool_f32(const Layer& L, const Tensor& x, Tensor& y) {
#pragma omp parallel for collapse(2)
    for (int b = 0; b < x.s.b; ++b)
        for (int c = 0; c < x.s.c; ++c)
            for (int oy = 0; oy < y.s.h; ++oy)
                for (int ox = 0; ox < y.s.w; ++ox) {
                    float acc = -std::numeric_limits<float>::infinity();
                    for (int ky = 0; ky < L.size; ++ky)
                        for (int kx = 0; kx < L.size; ++kx) {
                            int sy = oy * L.stride_y + ky - L.padding / 2;
                            int sx = ox * L.stride_x + kx - L.padding / 2;
                            if (sy < 0 || sy >= x.s.h || sx < 0 || sx >= x.s.w) continue;
                            acc = std::max(acc, x.d[x.off(b, c, sy, sx)]);
                        }
                    y.d[y.off(b, c, oy, ox)] = acc;
                }
}

// runtime/layer_ops.rs:1850-1883 forward_route
template <class T>
static void route_any(const Layer& L, const std::vector<T>& outs, T& y) {
    int oc = 0;
    for (int src : L.sources) {
        const T& s = outs[src];
        int chunk = s.s.c / std::max(L.route_groups, 1);
        int start = chunk * L.route_group_id;
        for (int b = 0; b < s.s.b; ++b)
            for (int c = 0; c < chunk; ++c)
                for (int yy = 0; yy < s.s.h; ++yy)
                    for (int xx = 0; xx < s.s.w; ++xx)
                        y.d[y.off(b, oc + c, yy, xx)] = s.d[s.off(b, start + c, yy, xx)];
        oc += chunk;
    }
}

// runtime/layer_ops.rs:2110-2145 forward_shortcut_with_cache: flat per-sample add of
// min(len) elements, activation after the last add.
static void shortcut_f32(const Layer& L, const Tensor& in, const std::vector<Tensor>& outs, Tensor& y) {
    y.d = in.d;
    for (int src : L.sources) {
        const Tensor& s = outs[src];
        if (s.s.b != y.s.b) throw std::runtime_error("shortcut mixes incompatible batch shapes");
        size_t os = y.s.count() / y.s.b, ss = s.s.count() / s.s.b, n = std::min(os, ss);
        for (int b = 0; b < y.s.b; ++b)
            for (size_t i = 0; i < n; ++i) y.d[b * os + i] += s.d[b * ss + i];
    }
    for (auto& v : y.d) v = activate(L.act, v);
}

// runtime/layer_ops.rs:2208-2256 forward_upsample
static void upsample_f32(const Layer& L, const Tensor& x, Tensor& y) {
    int st = L.up_stride;
    if (L.up_reverse) {
        std::fill(y.d.begin(), y.d.end(), 0.0f);
        int ch = y.s.h * st, cw = y.s.w * st;
        for (int b = 0; b < y.s.b; ++b)
            for (int c = 0; c < y.s.c; ++c)
                for (int yy = 0; yy < ch; ++yy)
                    for (int xx = 0; xx < cw; ++xx) y.d[y.off(b, c, yy / st, xx / st)] += L.up_scale * x.d[x.off(b, c, yy, xx)];
    } else {
        for (int b = 0; b < x.s.b; ++b)
            for (int c = 0; c < x.s.c; ++c)
                for (int yy = 0; yy < y.s.h; ++yy)
                    for (int xx = 0; xx < y.s.w; ++xx) y.d[y.off(b, c, yy, xx)] = L.up_scale * x.d[x.off(b, c, yy / st, xx / st)];
    }
}

static float amax_of(const std::vector<float>& v) {
    float m = 0.0f;
    for (float x : v) if (std::isfinite(x)) m = std::max(m, std::fabs(x));
    return m;
}

// runtime/exec_forward.rs:223-1100 layer walk (forward), f32.
// mode 0: faithful CPU path (unfolded BN); mode 1: BN folded first, like the GPU
// executor (runtime/gpu_params.rs:559-687).
static void forward_f32(Net& net, const float* input, int mode) {
    Shape is; is.w = net.width; is.h = net.height; is.c = net.channels; is.b = net.batch;
    Tensor cur(is);
    std::memcpy(cur.d.data(), input, cur.d.size() * sizeof(float));
    net.out_f32.assign(net.layers.size(), Tensor());
    net.amax.assign(net.layers.size() + 1, 0.0f);
    net.amax[0] = amax_of(cur.d);
    for (size_t i = 0; i < net.layers.size(); ++i) {
        Layer& L = net.layers[i];
        const Tensor& x = i == 0 ? cur : net.out_f32[i - 1];
        Tensor y(L.out);
        switch (L.kind) {
            case K_CONV: {
                if (mode == 1) {
                    std::vector<float> fw, fb;
                    fold_bn(L, x.s.c, fw, fb);
                    conv_f32(L, x, y, true, &fw, &fb);
                } else conv_f32(L, x, y, false, nullptr, nullptr);
                break;
            }
            case K_MAXPOOL: maxpool_f32(L, x, y); break;
            case K_ROUTE: route_any(L, net.out_f32, y); break;
            case K_SHORTCUT: shortcut_f32(L, x, net.out_f32, y); break;
            case K_UPSAMPLE: upsample_f32(L, x, y); break;
            case K_YOLO: y.d = x.d; break;  // exec_forward.rs:908-912 pass-through
        }
        net.amax[i + 1] = amax_of(y.d);
        net.out_f32[i] = std::move(y);
    }
}

// ---------------------------------------------------------------------------
// Deterministic transcendental: the int8/FP8 epilogues and the device decode use
// this exp instead of libm so that CPU and GPU agree bit for bit.  Every
// operation is a single IEEE-754 binary32 operation (fma where written), so any
// conforming implementation gives the same bits.  Accuracy: a few ulp of expf.
// ---------------------------------------------------------------------------

static inline float det_expf(float x) {
    x = std::fmin(std::fmax(x, -87.0f), 88.0f);
    const float LOG2E = 1.44269502e+00f;
    const float LN2_HI = 6.93145752e-01f;   // upper bits of ln 2
    const float LN2_LO = 1.42860677e-06f;   // ln 2 - LN2_HI
    float n = std::nearbyint(x * LOG2E);
    float r = std::fma(n, -LN2_HI, x);
    r = std::fma(n, -LN2_LO, r);
    float p = 1.98412698e-04f;               // 1/5040
    p = std::fma(p, r, 1.38888889e-03f);     // 1/720
    p = std::fma(p, r, 8.33333377e-03f);     // 1/120
    p = std::fma(p, r, 4.16666679e-02f);     // 1/24
    p = std::fma(p, r, 1.66666672e-01f);     // 1/6
    p = std::fma(p, r, 5.00000000e-01f);
    p = std::fma(p, r, 1.0f);
    p = std::fma(p, r, 1.0f);
    int32_t e = (int32_t)n;
    // 2^e as two factors so that e in [-126,127] never leaves the normal range.
    int32_t e1 = e / 2, e2 = e - e1;
    uint32_t b1 = (uint32_t)(e1 + 127) << 23, b2 = (uint32_t)(e2 + 127) << 23;
    float s1, s2;
    std::memcpy(&s1, &b1, 4);
    std::memcpy(&s2, &b2, 4);
    return p * s1 * s2;
}

static inline float det_sigmoid(float v) { return 1.0f / (1.0f + det_expf(-v)); }

// Activation of the quantised epilogue: same formulas as layer_ops.rs:1697-1738
// with exp replaced by det_expf and mish's tanh(ln(1+e^v)) rewritten as the
// algebraically equal w/(w+2), w = e^v(e^v+2).
static inline float det_activate(Act a, float v) {
    switch (a) {
        case ACT_LINEAR: return v;
        case ACT_LOGISTIC: return det_sigmoid(v);
        case ACT_RELU: return v > 0.0f ? v : 0.0f;
        case ACT_LEAKY: return v > 0.0f ? v : 0.1f * v;
        case ACT_MISH: {
            if (v > 20.0f) return v;
            float e = det_expf(v);
            float w = e * (e + 2.0f);
            return v * (w / (w + 2.0f));
        }
        case ACT_SWISH: return v / (1.0f + det_expf(-v));
    }
    return v;
}

// ---------------------------------------------------------------------------
// int8 model (defined by this build; the reference has none)
//   weights : per-output-channel symmetric, s_k = max|w_k|/127, q = rne(w/s_k) clamp +-127
//   tensors : per-tensor symmetric scale s = amax/127 from an f32 calibration run;
//             tensors joined by route / maxpool / upsample share one scale
//   conv    : acc = sum(xq*wq) int32;  v = fma(float(acc), s_x*s_k, b_k);  a = det_act(v)
//             int8 out: q = clamp(rne(a * (1/s_y)), +-127);  head conv (feeds [yolo]): a kept f32
// ---------------------------------------------------------------------------
// FP8 E4M3 codec: lightnet-cuda-oxide/src/fp8.rs:153-181 (RNE, satfinite 448,
// NaN -> 0x7F), decode :140-150.
// ---------------------------------------------------------------------------

static float e4m3_decode_mag(uint8_t m) {
    int e = (m >> 3) & 0xF, f = m & 7;
    if (e == 0) return std::ldexp((float)f, -9);
    return std::ldexp(1.0f + (float)f / 8.0f, e - 7);
}
static float e4m3_to_f32(uint8_t bits) {
    uint8_t m = bits & 0x7F;
    if (m == 0x7F) return std::numeric_limits<float>::quiet_NaN();
    float v = e4m3_decode_mag(m);
    return (bits & 0x80) ? -v : v;
}
static uint8_t f32_to_e4m3(float v) {
    if (std::isnan(v)) return 0x7F;
    uint8_t sign = std::signbit(v) ? 0x80 : 0;
    float mag = std::fabs(v);
    const uint8_t maxc = 0x7E;
    if (mag > e4m3_decode_mag(maxc)) return sign | maxc;
    uint8_t best = 0;
    float bd = std::numeric_limits<float>::infinity();
    for (int c = 0; c <= maxc; ++c) {
        float dist = std::fabs(mag - e4m3_decode_mag((uint8_t)c));
        if (dist < bd || (dist == bd && (c & 1) == 0)) { best = (uint8_t)c; bd = dist; }
    }
    return sign | best;
}


// Same mapping as f32_to_e4m3 (the reference's search), by binary search over the 127 finite magnitudes.
static uint8_t f32_to_e4m3_fast(float v) {
    static float mags[127];
    static bool init = false;
    if (!init) { for (int c = 0; c < 127; ++c) mags[c] = e4m3_decode_mag((uint8_t)c); init = true; }
    if (std::isnan(v)) return 0x7F;
    const uint8_t sign = std::signbit(v) ? 0x80 : 0;
    const float mag = std::fabs(v);
    if (mag > mags[126]) return sign | 0x7E;
    int hi = (int)(std::lower_bound(mags, mags + 127, mag) - mags);  // first code with magnitude >= mag
    if (hi == 0) return sign;
    const int lo = hi - 1;
    const float dl = mag - mags[lo], dh = mags[hi] - mag;
    int best = dl < dh ? lo : (dh < dl ? hi : ((lo & 1) == 0 ? lo : hi));
    return sign | (uint8_t)best;
}

// ---------------------------------------------------------------------------

static inline int8_t quant_i8(float a, float inv_s) {
    float r = std::nearbyint(a * inv_s);
    if (!(r >= -127.0f)) r = -127.0f;  // also maps NaN to -127
    if (r > 127.0f) r = 127.0f;
    return (int8_t)(int)r;
}

static void quantize_weights(Net& net) {
    for (size_t i = 0; i < net.layers.size(); ++i) {
        Layer& L = net.layers[i];
        if (L.kind != K_CONV) continue;
        std::vector<float> fw;
        fold_bn(L, L.in.c, fw, L.fbias);
        size_t per = fw.size() / L.filters;
        L.wq.assign(fw.size(), 0);
        L.wscale.assign(L.filters, 1.0f);
        for (int f = 0; f < L.filters; ++f) {
            float m = 0.0f;
            for (size_t k = 0; k < per; ++k) m = std::max(m, std::fabs(fw[f * per + k]));
            float s = (m > 0.0f && std::isfinite(m)) ? m / 127.0f : 1.0f;
            L.wscale[f] = s;
            for (size_t k = 0; k < per; ++k) L.wq[f * per + k] = quant_i8(fw[f * per + k] / s, 1.0f);
        }
        L.w8.assign(fw.size(), 0);
        L.w8scale.assign(L.filters, 1.0f);
        for (int f = 0; f < L.filters; ++f) {
            float m = 0.0f;
            for (size_t k = 0; k < per; ++k) m = std::max(m, std::fabs(fw[f * per + k]));
            float s8 = (m > 0.0f && std::isfinite(m)) ? m / 448.0f : 1.0f;
            L.w8scale[f] = s8;
            for (size_t k = 0; k < per; ++k) L.w8[f * per + k] = f32_to_e4m3_fast(fw[f * per + k] / s8);
        }
    }
}

struct UF {
    std::vector<int> p;
    explicit UF(int n) : p(n) { std::iota(p.begin(), p.end(), 0); }
    int find(int a) { while (p[a] != a) a = p[a] = p[p[a]]; return a; }
    void join(int a, int b) { a = find(a); b = find(b); if (a != b) p[std::max(a, b)] = std::min(a, b); }
};

// Scale groups: tensor index t = 0 is the network input, t = 1+i the output of layer i.
static void calibrate(Net& net, float qmax = 127.0f) {
    int T = (int)net.layers.size() + 1;
    UF uf(T);
    for (int i = 0; i < (int)net.layers.size(); ++i) {
        const Layer& L = net.layers[i];
        // tensors whose codes are copied share a scale; an up-sample that scales or sums (reverse) requantises instead
        if (L.kind == K_MAXPOOL || L.kind == K_YOLO || (L.kind == K_UPSAMPLE && !L.up_reverse && L.up_scale == 1.0f)) uf.join(i + 1, i);
        if (L.kind == K_ROUTE) for (int s : L.sources) uf.join(i + 1, s + 1);
    }
    std::vector<float> gmax(T, 0.0f);
    for (int t = 0; t < T; ++t) { int r = uf.find(t); gmax[r] = std::max(gmax[r], net.amax[t]); }
    net.scale.assign(T, 1.0f);
    for (int t = 0; t < T; ++t) {
        float m = gmax[uf.find(t)];
        net.scale[t] = (m > 0.0f && std::isfinite(m)) ? m / qmax : 1.0f;
    }
}

static bool feeds_head(const Net& net, int i) {
    // runtime/types.rs:146-170 conv_feeds_detection_head
    return net.layers[i].kind == K_CONV && i + 1 < (int)net.layers.size() && net.layers[i + 1].kind == K_YOLO;
}

// int32 accumulators of one int8 conv; NCHW in, NCHW out.  Integer arithmetic is
// order independent, so any loop order is exact.
// `groups`: filter f reads the C / groups channels of group f / (F / groups), as forward_layers.rs:646-679 does
// (input channel g * cpg + ic, weight [f][ic][ky][kx]).
static void conv_q8_acc(const int8_t* x, int B, int C, int H, int W, const int8_t* wq, int F, int k, int sx, int sy,
                        int pad, int OH, int OW, int32_t* acc, int groups = 1) {
    const int cpg = C / groups, fpg = F / groups;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; ++b)
        for (int f = 0; f < F; ++f) {
            int32_t* out = acc + ((size_t)b * F + f) * OH * OW;
            std::fill(out, out + (size_t)OH * OW, 0);
            for (int ic = 0; ic < cpg; ++ic) {
                const int8_t* xp = x + ((size_t)b * C + (f / fpg) * cpg + ic) * H * W;
                for (int ky = 0; ky < k; ++ky)
                    for (int kx = 0; kx < k; ++kx) {
                        int32_t wv = wq[(((size_t)f * cpg + ic) * k + ky) * k + kx];
                        if (wv == 0) continue;
                        for (int oy = 0; oy < OH; ++oy) {
                            int yy = oy * sy + ky - pad;
                            if (yy < 0 || yy >= H) continue;
                            const int8_t* row = xp + (size_t)yy * W;
                            int32_t* orow = out + (size_t)oy * OW;
                            for (int ox = 0; ox < OW; ++ox) {
                                int xx = ox * sx + kx - pad;
                                if (xx < 0 || xx >= W) continue;
                                orow[ox] += wv * (int32_t)row[xx];
                            }
                        }
                    }
            }
        }
}

static void forward_q8(Net& net, const float* input) {
    const int NL = (int)net.layers.size();
    net.out_q8.assign(NL, TensorI8());
    net.head_q8.assign(NL, Tensor());
    Shape is; is.w = net.width; is.h = net.height; is.c = net.channels; is.b = net.batch;
    TensorI8 xin(is);
    {
        float inv = 1.0f / net.scale[0];
        for (size_t i = 0; i < xin.d.size(); ++i) xin.d[i] = quant_i8(input[i], inv);
    }
    for (int i = 0; i < NL; ++i) {
        Layer& L = net.layers[i];
        const TensorI8& x = i == 0 ? xin : net.out_q8[i - 1];
        const float sx = net.scale[i], sy = net.scale[i + 1];  // scale[i] = scale of layer i-1's output
        TensorI8 y(L.out);
        switch (L.kind) {
            case K_CONV: {
                if (L.dilation != 1) throw std::runtime_error("int8 conv supports dilation=1");
                std::vector<int32_t> acc(L.out.count());
                conv_q8_acc(x.d.data(), x.s.b, x.s.c, x.s.h, x.s.w, L.wq.data(), L.filters, L.size, L.stride_x, L.stride_y,
                            L.padding, L.out.h, L.out.w, acc.data(), std::max(L.groups, 1));
                bool head = feeds_head(net, i);
                if (head) net.head_q8[i] = Tensor(L.out);
                float inv = 1.0f / sy;
                size_t plane = (size_t)L.out.h * L.out.w;
                for (int b = 0; b < L.out.b; ++b)
                    for (int f = 0; f < L.filters; ++f) {
                        float m = sx * L.wscale[f];
                        float bias = L.fbias[f];
                        size_t base = ((size_t)b * L.filters + f) * plane;
                        for (size_t p = 0; p < plane; ++p) {
                            float v = std::fma((float)acc[base + p], m, bias);
                            float a = det_activate(L.act, v);
                            if (head) net.head_q8[i].d[base + p] = a;
                            else y.d[base + p] = quant_i8(a, inv);
                        }
                    }
                break;
            }
            case K_MAXPOOL: {
                for (int b = 0; b < x.s.b; ++b)
                    for (int c = 0; c < x.s.c; ++c)
                        for (int oy = 0; oy < y.s.h; ++oy)
                            for (int ox = 0; ox < y.s.w; ++ox) {
                                int m = -127;
                                for (int ky = 0; ky < L.size; ++ky)
                                    for (int kx = 0; kx < L.size; ++kx) {
                                        int yy = oy * L.stride_y + ky - L.padding / 2;
                                        int xx = ox * L.stride_x + kx - L.padding / 2;
                                        if (yy < 0 || yy >= x.s.h || xx < 0 || xx >= x.s.w) continue;
                                        m = std::max(m, (int)x.d[x.off(b, c, yy, xx)]);
                                    }
                                y.d[y.off(b, c, oy, ox)] = (int8_t)m;
                            }
                break;
            }
            case K_ROUTE: route_any(L, net.out_q8, y); break;
            case K_SHORTCUT: {
                float inv = 1.0f / sy;
                // a source of another shape is cropped / zero-padded flat per sample (lib.rs:4041 shortcut_fit, layer_ops.rs:2110-2145):
                // element p of a sample takes the source's element p while the source has one
                const size_t os = y.s.count() / y.s.b;
                for (size_t p = 0; p < y.d.size(); ++p) {
                    const size_t b = p / os, q = p % os;
                    float v = (float)x.d[p] * sx;
                    for (int src : L.sources) {
                        const TensorI8& sT = net.out_q8[src];
                        if (sT.s.b != y.s.b) throw std::runtime_error("shortcut mixes incompatible batch shapes");
                        const size_t ss = sT.s.count() / sT.s.b;
                        v = std::fma(q < ss ? (float)sT.d[b * ss + q] : 0.0f, net.scale[src + 1], v);
                    }
                    y.d[p] = quant_i8(det_activate(L.act, v), inv);
                }
                break;
            }
            case K_UPSAMPLE: {
                const int st = L.up_stride;
                if (!L.up_reverse && L.up_scale == 1.0f) {  // codes copied, scale shared
                    for (int b = 0; b < y.s.b; ++b)
                        for (int c = 0; c < y.s.c; ++c)
                            for (int yy = 0; yy < y.s.h; ++yy)
                                for (int xx = 0; xx < y.s.w; ++xx)
                                    y.d[y.off(b, c, yy, xx)] = x.d[x.off(b, c, yy / st, xx / st)];
                    break;
                }
                // layer_ops.rs:2208-2256 on codes: out = scale * in (nearest) or scale * sum of the stride x stride block (reverse; the
                // integer sum is exact, taken in (dy, dx) order), requantised with r = s_in * scale / s_out
                const float r = (sx * L.up_scale) / sy;
                for (int b = 0; b < y.s.b; ++b)
                    for (int c = 0; c < y.s.c; ++c)
                        for (int yy = 0; yy < y.s.h; ++yy)
                            for (int xx = 0; xx < y.s.w; ++xx) {
                                float v;
                                if (L.up_reverse) {
                                    int sum = 0;
                                    for (int dy = 0; dy < st; ++dy)
                                        for (int dx = 0; dx < st; ++dx) {
                                            const int iy = yy * st + dy, ix = xx * st + dx;
                                            if (iy < x.s.h && ix < x.s.w) sum += x.d[x.off(b, c, iy, ix)];
                                        }
                                    v = (float)sum;
                                } else v = (float)x.d[x.off(b, c, yy / st, xx / st)];
                                y.d[y.off(b, c, yy, xx)] = quant_i8(v, r);
                            }
                break;
            }
            case K_YOLO: {
                if (i == 0 || !feeds_head(net, i - 1)) throw std::runtime_error("int8 [yolo] must follow a convolution");
                net.head_q8[i] = net.head_q8[i - 1];
                break;
            }
        }
        net.out_q8[i] = std::move(y);
    }
}

// FP8 E4M3 forward: the int8 model with E4M3 codes (scales amax/448, lightnet-cuda-oxide/src/fp8.rs:186) and
// floating-point accumulation.  Accumulation is done in double here; a tensor core accumulates in f32 in its own
// order, so comparisons against this are toleranced, never bit-exact.
static inline int8_t f8_key(uint8_t c) { return (int8_t)((c & 0x80) ? (c ^ 0x7F) : c); }  // order of the values under signed compare

static void forward_f8(Net& net, const float* input) {
    const int NL = (int)net.layers.size();
    net.out_f8.assign(NL, std::vector<uint8_t>());
    net.head_f8.assign(NL, Tensor());
    Shape is; is.w = net.width; is.h = net.height; is.c = net.channels; is.b = net.batch;
    std::vector<uint8_t> xin(is.count());
    {
        float inv = 1.0f / net.scale[0];
        for (size_t i = 0; i < xin.size(); ++i) xin[i] = f32_to_e4m3_fast(input[i] * inv);
    }
    auto off = [](const Shape& s, int b, int c, int y, int x) { return (((size_t)b * s.c + c) * s.h + y) * s.w + x; };
    float dec[256];
    for (int c = 0; c < 256; ++c) dec[c] = ((c & 0x7F) == 0x7F) ? 0.0f : e4m3_to_f32((uint8_t)c);
    for (int i = 0; i < NL; ++i) {
        Layer& L = net.layers[i];
        const std::vector<uint8_t>& x = i == 0 ? xin : net.out_f8[i - 1];
        const Shape xs = L.in;
        const float sx = net.scale[i], sy = net.scale[i + 1];
        std::vector<uint8_t> y(L.out.count(), 0);
        switch (L.kind) {
            case K_CONV: {
                if (L.groups != 1 || L.dilation != 1) throw std::runtime_error("fp8 conv supports groups=1 dilation=1");
                const bool head = feeds_head(net, i);
                if (head) net.head_f8[i] = Tensor(L.out);
                const float inv = 1.0f / sy;
                const int C = xs.c, k = L.size;
#pragma omp parallel for collapse(2) schedule(dynamic)
                for (int b = 0; b < L.out.b; ++b)
                    for (int f = 0; f < L.filters; ++f) {
                        const float m = sx * L.w8scale[f], bias = L.fbias[f];
                        for (int oy = 0; oy < L.out.h; ++oy)
                            for (int ox = 0; ox < L.out.w; ++ox) {
                                double acc = 0.0;
                                for (int ic = 0; ic < C; ++ic)
                                    for (int ky = 0; ky < k; ++ky) {
                                        const int yy = oy * L.stride_y + ky - L.padding;
                                        if (yy < 0 || yy >= xs.h) continue;
                                        for (int kx = 0; kx < k; ++kx) {
                                            const int xx = ox * L.stride_x + kx - L.padding;
                                            if (xx < 0 || xx >= xs.w) continue;
                                            acc += (double)dec[x[off(xs, b, ic, yy, xx)]] * (double)dec[L.w8[(((size_t)f * C + ic) * k + ky) * k + kx]];
                                        }
                                    }
                                const float a = det_activate(L.act, std::fma((float)acc, m, bias));
                                const size_t o = off(L.out, b, f, oy, ox);
                                if (head) net.head_f8[i].d[o] = a;
                                else y[o] = f32_to_e4m3_fast(a * inv);
                            }
                    }
                break;
            }
            case K_MAXPOOL:
                for (int b = 0; b < xs.b; ++b)
                    for (int c = 0; c < xs.c; ++c)
                        for (int oy = 0; oy < L.out.h; ++oy)
                            for (int ox = 0; ox < L.out.w; ++ox) {
                                uint8_t best = 0xFE;
                                for (int ky = 0; ky < L.size; ++ky)
                                    for (int kx = 0; kx < L.size; ++kx) {
                                        const int yy = oy * L.stride_y + ky - L.padding / 2, xx = ox * L.stride_x + kx - L.padding / 2;
                                        if (yy < 0 || yy >= xs.h || xx < 0 || xx >= xs.w) continue;
                                        const uint8_t v = x[off(xs, b, c, yy, xx)];
                                        if (f8_key(v) > f8_key(best)) best = v;
                                    }
                                y[off(L.out, b, c, oy, ox)] = best;
                            }
                break;
            case K_ROUTE: {
                int oc = 0;
                for (int src : L.sources) {
                    const Shape ss = net.layers[src].out;
                    const int chunk = ss.c / std::max(L.route_groups, 1), start = chunk * L.route_group_id;
                    for (int b = 0; b < ss.b; ++b)
                        for (int c = 0; c < chunk; ++c)
                            for (int yy = 0; yy < ss.h; ++yy)
                                for (int xx = 0; xx < ss.w; ++xx) y[off(L.out, b, oc + c, yy, xx)] = net.out_f8[src][off(ss, b, start + c, yy, xx)];
                    oc += chunk;
                }
                break;
            }
            case K_SHORTCUT: {
                const float inv = 1.0f / sy;
                for (int src : L.sources)
                    if (net.layers[src].out.count() != L.out.count()) throw std::runtime_error("fp8 shortcut needs same-shape sources");
                for (size_t p = 0; p < y.size(); ++p) {
                    float v = dec[x[p]] * sx;
                    for (int src : L.sources) v = std::fma(dec[net.out_f8[src][p]], net.scale[src + 1], v);
                    y[p] = f32_to_e4m3_fast(det_activate(L.act, v) * inv);
                }
                break;
            }
            case K_UPSAMPLE:
                if (L.up_reverse || L.up_scale != 1.0f) throw std::runtime_error("fp8 upsample supports scale=1, forward only");
                for (int b = 0; b < L.out.b; ++b)
                    for (int c = 0; c < L.out.c; ++c)
                        for (int yy = 0; yy < L.out.h; ++yy)
                            for (int xx = 0; xx < L.out.w; ++xx) y[off(L.out, b, c, yy, xx)] = x[off(xs, b, c, yy / L.up_stride, xx / L.up_stride)];
                break;
            case K_YOLO:
                if (i == 0 || !feeds_head(net, i - 1)) throw std::runtime_error("fp8 [yolo] must follow a convolution");
                net.head_f8[i] = net.head_f8[i - 1];
                break;
        }
        net.out_f8[i] = std::move(y);
    }
}

// ---------------------------------------------------------------------------
// Decode + NMS
// ---------------------------------------------------------------------------

struct Det {
    int class_id;
    float conf, obj, x, y, w, h;
};

// lightnet-model/src/detection_geometry.rs:80-102 (sigmoid/head_activation)
static inline float head_act(float raw, bool new_coords, bool det) {
    if (new_coords) return raw;
    return det ? det_sigmoid(raw) : 1.0f / (1.0f + std::exp(-raw));
}

struct HeadSpec {
    int gw, gh, classes, n_anchor;
    const float* anchors_wh;  // n_anchor pairs, already selected through mask
    float scale_x_y;
    int new_coords;
    // 0 = [yolo] / [gaussian_yolo]; 1 = activated [yolox] head (classes + 5 channels, cxcywh logits); 2 = a distribution head
    // ([ppyoloe], [yolonas]) after modern_yolo_predecode: final centre-size box, objectness, classes
    int kind = 0;
};

static inline float finite_or_zero(float v) { return std::isfinite(v) ? v : 0.0f; }
static inline float clamp01(float v) { return std::min(std::max(v, 0.0f), 1.0f); }

// lightnet-train/src/detect.rs:1035-1125 decode_modern_detections (the candidates of one image's head, before its NMS), with
// lightnet-layers/src/modern_yolo/cpu.rs:461-475 decode_yolox_box, :493-527 modern_objectness / modern_class_score and
// detect.rs:1414-1447 correct_bbox.  The emission order is (cell, class), as the reference's loops run.
static void decode_modern_head(const float* data, const HeadSpec& hs, int net_w, int net_h, int img_w, int img_h, float thr,
                               bool letterbox, bool det_exp, std::vector<Det>& out) {
    const int stride = hs.gw * hs.gh;
    const float iw = (float)img_w, ih = (float)img_h, nw = (float)net_w, nh = (float)net_h;
    float new_w, new_h;
    if (letterbox) {
        if (nw / iw < nh / ih) { new_w = nw; new_h = ih * nw / iw; }
        else { new_w = iw * nh / ih; new_h = nh; }
    } else { new_w = nw; new_h = nh; }
    const float delta_w = nw - new_w, delta_h = nh - new_h, ratio_w = new_w / nw, ratio_h = new_h / nh;
    for (int idx = 0; idx < stride; ++idx) {
        const int row = idx / hs.gw, col = idx % hs.gw;
        const float obj = clamp01(finite_or_zero(data[(size_t)4 * stride + idx]));
        bool have = false;
        float bx = 0, by = 0, bw = 0, bh = 0;
        for (int c = 0; c < hs.classes; ++c) {
            const float cls = clamp01(finite_or_zero(data[(size_t)(5 + c) * stride + idx]));
            // the distribution heads gate on the class score, not on the product (detect.rs:1158-1162)
            const float score = hs.kind == 2 ? std::max(cls, obj * cls) : obj * cls;
            if (score <= thr) continue;
            if (!have) {
                have = true;
                if (hs.kind == 2) {
                    bx = data[idx]; by = data[(size_t)stride + idx]; bw = data[(size_t)2 * stride + idx]; bh = data[(size_t)3 * stride + idx];
                } else {
                    const float tw = std::min(std::max(finite_or_zero(data[(size_t)2 * stride + idx]), -10.0f), 10.0f);
                    const float th = std::min(std::max(finite_or_zero(data[(size_t)3 * stride + idx]), -10.0f), 10.0f);
                    bx = ((float)col + finite_or_zero(data[idx])) / (float)hs.gw;
                    by = ((float)row + finite_or_zero(data[(size_t)stride + idx])) / (float)hs.gh;
                    bw = (det_exp ? det_expf(tw) : std::exp(tw)) / (float)hs.gw;
                    bh = (det_exp ? det_expf(th) : std::exp(th)) / (float)hs.gh;
                    bx = finite_or_zero(bx); by = finite_or_zero(by);                                      // sanitize (cpu.rs:212-217)
                    bw = std::max(finite_or_zero(bw), 1e-6f); bh = std::max(finite_or_zero(bh), 1e-6f);
                }
                bx = (bx - delta_w / 2.0f / nw) / ratio_w;
                by = (by - delta_h / 2.0f / nh) / ratio_h;
                bw /= ratio_w;
                bh /= ratio_h;
                bx *= iw; by *= ih; bw *= iw; bh *= ih;
            }
            out.push_back(Det{c, score, obj, bx, by, bw, bh});
        }
    }
}

// lightnet-train/src/detect.rs:934-1016 decode_yolo_head, :1288-1322 decode_bbox,
// :1414-1447 correct_bbox.  `data` is one image's head, channel-major
// [anchor*(5+classes)+entry][gh*gw].  det_exp selects det_expf instead of libm.
static void decode_head(const float* data, const HeadSpec& hs, int net_w, int net_h, int img_w, int img_h, float thr,
                        bool letterbox, bool det_exp, std::vector<Det>& out) {
    if (hs.kind != 0) { decode_modern_head(data, hs, net_w, net_h, img_w, img_h, thr, letterbox, det_exp, out); return; }
    const int stride = hs.gw * hs.gh, epa = hs.classes + 5;
    const bool nc = hs.new_coords != 0;
    const float iw = (float)img_w, ih = (float)img_h, nw = (float)net_w, nh = (float)net_h;
    float new_w, new_h;
    if (letterbox) {
        if (nw / iw < nh / ih) { new_w = nw; new_h = ih * nw / iw; }
        else { new_w = iw * nh / ih; new_h = nh; }
    } else { new_w = nw; new_h = nh; }
    const float delta_w = nw - new_w, delta_h = nh - new_h, ratio_w = new_w / nw, ratio_h = new_h / nh;
    for (int a = 0; a < hs.n_anchor; ++a) {
        const float aw = hs.anchors_wh[2 * a], ah = hs.anchors_wh[2 * a + 1];
        const int ab = a * epa;
        for (int idx = 0; idx < stride; ++idx) {
            const int row = idx / hs.gw, col = idx % hs.gw;
            float tx = data[(size_t)(ab + 0) * stride + idx];
            float ty = data[(size_t)(ab + 1) * stride + idx];
            float tw = data[(size_t)(ab + 2) * stride + idx];
            float th = data[(size_t)(ab + 3) * stride + idx];
            float obj = head_act(data[(size_t)(ab + 4) * stride + idx], nc, det_exp);
            if (obj <= thr) continue;
            float bx = ((float)col + hs.scale_x_y * head_act(tx, nc, det_exp) - 0.5f * (hs.scale_x_y - 1.0f)) / (float)hs.gw;
            float by = ((float)row + hs.scale_x_y * head_act(ty, nc, det_exp) - 0.5f * (hs.scale_x_y - 1.0f)) / (float)hs.gh;
            float bw, bh;
            if (nc) { bw = tw * tw * 4.0f * aw / nw; bh = th * th * 4.0f * ah / nh; }
            else {
                bw = (det_exp ? det_expf(tw) : std::exp(tw)) * aw / nw;
                bh = (det_exp ? det_expf(th) : std::exp(th)) * ah / nh;
            }
            bx = (bx - delta_w / 2.0f / nw) / ratio_w;
            by = (by - delta_h / 2.0f / nh) / ratio_h;
            bw /= ratio_w;
            bh /= ratio_h;
            bx *= iw; by *= ih; bw *= iw; bh *= ih;
            for (int c = 0; c < hs.classes; ++c) {
                float p = head_act(data[(size_t)(ab + 5 + c) * stride + idx], nc, det_exp);
                float conf = obj * p;
                if (conf > thr) out.push_back(Det{c, conf, obj, bx, by, bw, bh});
            }
        }
    }
}

// lightnet-train/src/detect.rs:1486-1503 bbox_iou; detection_geometry.rs:14-30 edges
static inline float bbox_iou(const Det& a, const Det& b) {
    float al = a.x - a.w * 0.5f, at = a.y - a.h * 0.5f, ar = a.x + a.w * 0.5f, ab = a.y + a.h * 0.5f;
    float bl = b.x - b.w * 0.5f, bt = b.y - b.h * 0.5f, br = b.x + b.w * 0.5f, bb = b.y + b.h * 0.5f;
    float il = std::max(al, bl), it = std::max(at, bt), ir = std::min(ar, br), ib = std::min(ab, bb);
    float iw = std::max(ir - il, 0.0f), ih = std::max(ib - it, 0.0f);
    float inter = iw * ih;
    if (inter <= 0.0f) return 0.0f;
    float aa = std::max(a.w, 0.0f) * std::max(a.h, 0.0f), ba = std::max(b.w, 0.0f) * std::max(b.h, 0.0f);
    return inter / (aa + ba - inter);
}

// lightnet-train/src/detect.rs:1449-1484 apply_nms.  The survivor compaction there
// swaps survivors forward, which keeps survivors in their original relative order.
static void apply_nms(std::vector<Det>& d, float thr) {
    if (thr <= 0.0f) return;
    const size_t n = d.size();
    std::vector<char> sup(n, 0);
    for (size_t i = 0; i < n; ++i) {
        if (sup[i]) continue;
        for (size_t j = i + 1; j < n; ++j) {
            if (sup[j] || d[i].class_id != d[j].class_id) continue;
            size_t keep, drop;
            if (d[i].conf >= d[j].conf) { keep = i; drop = j; } else { keep = j; drop = i; }
            if (bbox_iou(d[keep], d[drop]) > thr) sup[drop] = 1;
        }
    }
    size_t k = 0;
    for (size_t i = 0; i < n; ++i) if (!sup[i]) { if (k != i) d[k] = d[i]; ++k; }
    d.resize(k);
}

// f32::total_cmp descending, stable (detect.rs:107, :242)
static void sort_conf_desc(std::vector<Det>& d) {
    auto key = [](float f) { int32_t b; std::memcpy(&b, &f, 4); return b < 0 ? (int32_t)(b ^ 0x7fffffff) : b; };
    std::stable_sort(d.begin(), d.end(), [&](const Det& a, const Det& b) { return key(a.conf) > key(b.conf); });
}

// lightnet-train/src/detect.rs:113-244 decode_network_detections for one image:
// all heads decoded (emission order head, anchor, cell, class); apply_nms(1.0) on the
// unsorted list; stable sort; apply_nms(nms_thr); stable sort.  `skip_pass1` drops the
// thr=1.0 pass (used by tests to show it is a no-op on a given input).  top_k > 0
// truncates the final list (an extension; the reference has no top-k).
static std::vector<Det> detect_image(const std::vector<const float*>& heads, const std::vector<HeadSpec>& specs, int net_w,
                                     int net_h, int img_w, int img_h, float thr, float nms_thr, bool letterbox, int top_k,
                                     bool det_exp, bool skip_pass1) {
    std::vector<Det> d;
    for (size_t h = 0; h < heads.size(); ++h) decode_head(heads[h], specs[h], net_w, net_h, img_w, img_h, thr, letterbox, det_exp, d);
    if (!skip_pass1) apply_nms(d, 1.0f);
    sort_conf_desc(d);
    apply_nms(d, nms_thr);
    sort_conf_desc(d);
    if (top_k > 0 && (int)d.size() > top_k) d.resize(top_k);
    return d;
}

}  // namespace orc

// ---------------------------------------------------------------------------
// C API (ctypes)
// ---------------------------------------------------------------------------

using namespace orc;

static thread_local std::string g_err;

#define ORC_TRY try {
#define ORC_CATCH(ret) } catch (const std::exception& e) { g_err = e.what(); return ret; }

extern "C" {

const char* orc_last_error() { return g_err.c_str(); }

void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
int orc_max_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void* orc_net_create(const char* cfg_text, int batch) {
    ORC_TRY
    return build_net(cfg_text, batch).release();
    ORC_CATCH(nullptr)
}
void orc_net_destroy(void* h) { delete (Net*)h; }
int orc_net_num_layers(void* h) { return (int)((Net*)h)->layers.size(); }

// info[16]: kind, in(w,h,c,b), out(w,h,c,b), filters,size,stride_x,stride_y,padding,bn,act
int orc_net_layer_info(void* h, int i, int* info) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->layers.size()) return -1;
    const Layer& L = n->layers[i];
    int v[20] = {L.kind, L.in.w, L.in.h, L.in.c, L.in.b, L.out.w, L.out.h, L.out.c, L.out.b,
                 L.filters, L.size, L.stride_x, L.stride_y, L.padding, L.bn ? 1 : 0, (int)L.act, std::max(L.groups, 1), std::max(L.dilation, 1), 0, 0};
    std::memcpy(info, v, sizeof v);
    return 0;
}
// Absolute source layers of a route / shortcut; yolo: mask entries.  Returns the count.
int orc_net_layer_sources(void* h, int i, int* out, int max_out) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->layers.size()) return -1;
    const Layer& L = n->layers[i];
    const std::vector<int>& v = L.kind == K_YOLO ? L.mask : L.sources;
    for (int k = 0; k < (int)v.size() && k < max_out; ++k) out[k] = v[k];
    return (int)v.size();
}
void orc_net_dims(void* h, int* whcb) {
    Net* n = (Net*)h;
    whcb[0] = n->width; whcb[1] = n->height; whcb[2] = n->channels; whcb[3] = n->batch;
}

// Darknet .weights payload order (runtime/weights_io.rs:227-235): per conv biases,
// [scales, rolling_mean, rolling_variance], weights.
long long orc_net_weight_count(void* h) {
    long long c = 0;
    for (auto& L : ((Net*)h)->layers)
        if (L.kind == K_CONV) c += (long long)L.biases.size() * (L.bn ? 4 : 1) + (long long)L.weights.size();
    return c;
}
int orc_net_set_weights(void* h, const float* w, long long count) {
    ORC_TRY
    Net* n = (Net*)h;
    if (count != orc_net_weight_count(h)) throw std::runtime_error("weight count mismatch");
    for (auto& L : n->layers) {
        if (L.kind != K_CONV) continue;
        auto take = [&](std::vector<float>& v) { std::memcpy(v.data(), w, v.size() * 4); w += v.size(); };
        take(L.biases);
        if (L.bn) { take(L.scales); take(L.mean); take(L.var); }
        take(L.weights);
    }
    quantize_weights(*n);
    return 0;
    ORC_CATCH(-1)
}

int orc_net_forward_f32(void* h, const float* input, int mode) {
    ORC_TRY
    forward_f32(*(Net*)h, input, mode);
    return 0;
    ORC_CATCH(-1)
}
int orc_net_layer_output_f32(void* h, int i, float* out) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->out_f32.size()) return -1;
    std::memcpy(out, n->out_f32[i].d.data(), n->out_f32[i].d.size() * 4);
    return 0;
}
int orc_net_calibrate(void* h) {
    ORC_TRY
    Net* n = (Net*)h;
    if (n->amax.size() != n->layers.size() + 1) throw std::runtime_error("run forward_f32 before calibrate");
    calibrate(*n);
    return 0;
    ORC_CATCH(-1)
}
// amax / scale arrays have num_layers+1 entries: [0] input, [1+i] layer i output.
int orc_net_get_amax(void* h, float* out) {
    Net* n = (Net*)h;
    std::memcpy(out, n->amax.data(), n->amax.size() * 4);
    return (int)n->amax.size();
}
int orc_net_get_scales(void* h, float* out) {
    Net* n = (Net*)h;
    std::memcpy(out, n->scale.data(), n->scale.size() * 4);
    return (int)n->scale.size();
}
int orc_net_set_scales(void* h, const float* s, int count) {
    Net* n = (Net*)h;
    if (count != (int)n->layers.size() + 1) return -1;
    n->scale.assign(s, s + count);
    return 0;
}
int orc_net_calibrate_qmax(void* h, float qmax) {
    ORC_TRY
    Net* n = (Net*)h;
    if (n->amax.size() != n->layers.size() + 1) throw std::runtime_error("run forward_f32 before calibrate");
    calibrate(*n, qmax);
    return 0;
    ORC_CATCH(-1)
}
int orc_net_forward_f8(void* h, const float* input) {
    ORC_TRY
    Net* n = (Net*)h;
    if (n->scale.size() != n->layers.size() + 1) throw std::runtime_error("scales are not set");
    forward_f8(*n, input);
    return 0;
    ORC_CATCH(-1)
}
int orc_net_layer_output_f8(void* h, int i, uint8_t* out) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->out_f8.size()) return -1;
    std::memcpy(out, n->out_f8[i].data(), n->out_f8[i].size());
    return 0;
}
int orc_net_head_f8(void* h, int i, float* out) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->head_f8.size() || n->head_f8[i].d.empty()) return -1;
    std::memcpy(out, n->head_f8[i].d.data(), n->head_f8[i].d.size() * 4);
    return 0;
}
unsigned char orc_f32_to_e4m3_fast(float v) { return f32_to_e4m3_fast(v); }
int orc_net_forward_q8(void* h, const float* input) {
    ORC_TRY
    Net* n = (Net*)h;
    if (n->scale.size() != n->layers.size() + 1) throw std::runtime_error("scales are not set");
    forward_q8(*n, input);
    return 0;
    ORC_CATCH(-1)
}
int orc_net_layer_output_q8(void* h, int i, int8_t* out) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->out_q8.size()) return -1;
    std::memcpy(out, n->out_q8[i].d.data(), n->out_q8[i].d.size());
    return 0;
}
// f32 head of the int8 run; i = the [yolo] layer index (or its conv).
int orc_net_head_q8(void* h, int i, float* out) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->head_q8.size() || n->head_q8[i].d.empty()) return -1;
    std::memcpy(out, n->head_q8[i].d.data(), n->head_q8[i].d.size() * 4);
    return 0;
}
// Per-filter weight scale and quantised weights of conv layer i.
int orc_net_conv_quant(void* h, int i, int8_t* wq, float* wscale, float* fbias) {
    Net* n = (Net*)h;
    if (i < 0 || i >= (int)n->layers.size() || n->layers[i].kind != K_CONV) return -1;
    const Layer& L = n->layers[i];
    if (wq) std::memcpy(wq, L.wq.data(), L.wq.size());
    if (wscale) std::memcpy(wscale, L.wscale.data(), L.wscale.size() * 4);
    if (fbias) std::memcpy(fbias, L.fbias.data(), L.fbias.size() * 4);
    return 0;
}

// Detections of image `b` from the last run (source 0 = f32 run, 1 = int8 run).
// out: records of 7 floats {class, conf, obj, x, y, w, h}; returns the count (may
// exceed max_out; only max_out are written) or -1.
int orc_net_detect(void* h, int source, int b, int img_w, int img_h, float thr, float nms_thr, int letterbox, int top_k,
                   int det_exp, int skip_pass1, float* out, int max_out) {
    ORC_TRY
    Net* n = (Net*)h;
    std::vector<const float*> heads;
    std::vector<HeadSpec> specs;
    std::vector<std::vector<float>> anch;
    for (size_t i = 0; i < n->layers.size(); ++i) {
        const Layer& L = n->layers[i];
        if (L.kind != K_YOLO) continue;
        const Tensor& t = source == 0 ? n->out_f32[i] : n->head_q8[i];
        if (t.d.empty()) throw std::runtime_error("no head output; run forward first");
        size_t sample = (size_t)t.s.w * t.s.h * L.mask.size() * (L.classes + 5);
        if (sample * t.s.b != t.d.size()) throw std::runtime_error("YOLO head tensor length mismatch");
        if (b < 0 || b >= t.s.b) throw std::runtime_error("batch index outside YOLO head batch");
        heads.push_back(t.d.data() + sample * b);
        std::vector<float> a;
        for (int m : L.mask) {
            if ((size_t)(2 * m + 1) >= L.anchors.size()) throw std::runtime_error("missing anchor for YOLO mask index");
            a.push_back(L.anchors[2 * m]);
            a.push_back(L.anchors[2 * m + 1]);
        }
        anch.push_back(a);
        HeadSpec hs;
        hs.gw = t.s.w; hs.gh = t.s.h; hs.classes = L.classes; hs.n_anchor = (int)L.mask.size();
        hs.anchors_wh = nullptr; hs.scale_x_y = L.scale_x_y; hs.new_coords = L.new_coords;
        specs.push_back(hs);
    }
    for (size_t k = 0; k < specs.size(); ++k) specs[k].anchors_wh = anch[k].data();
    auto d = detect_image(heads, specs, n->width, n->height, img_w, img_h, thr, nms_thr, letterbox != 0, top_k, det_exp != 0,
                          skip_pass1 != 0);
    for (int i = 0; i < (int)d.size() && i < max_out; ++i) {
        float* r = out + 7 * i;
        r[0] = (float)d[i].class_id; r[1] = d[i].conf; r[2] = d[i].obj; r[3] = d[i].x; r[4] = d[i].y; r[5] = d[i].w; r[6] = d[i].h;
    }
    return (int)d.size();
    ORC_CATCH(-1)
}

// lightnet-cuda/src/lib.rs:4884-4915 modern_yolo_forward_f32 (= modern_yolo/cpu.rs:268-281 activate_modern_output): every entry
// sanitised, the trailing 1 + classes planes through a sigmoid of the logit clamped to [-30, 30].  In place, NCHW.
int orc_modern_activate(float* x, int batch, int channels, int spatial, int classes) {
    const int class_begin = std::max(channels - (classes + 1), 0);
    for (int b = 0; b < batch; ++b)
        for (int c = 0; c < channels; ++c)
            for (int i = 0; i < spatial; ++i) {
                float& v = x[((size_t)b * channels + c) * spatial + i];
                if (!std::isfinite(v)) v = 0.0f;
                if (c >= class_begin) v = 1.0f / (1.0f + std::exp(-std::min(std::max(v, -30.0f), 30.0f)));
            }
    return 0;
}

// lightnet-cuda-oxide/src/kernels/dense_loss.rs:788-812 modern_yolo_predecode with modern_yolo/cpu.rs:283-308 dfl_expectation,
// :340-362 box_from_corners, :364-387 decode_dfl_box: an activated [ppyoloe] / [yolonas] head [batch, coords + 1 + classes, h, w]
// -> [batch, 5 + classes, h, w]: the final centre-size box, then the objectness and class planes copied.
int orc_modern_predecode(const float* act, float* out, int batch, int w, int h, int classes, int coords) {
    const int s = w * h, bins = std::max(coords / 4, 2), cin = coords + 1 + classes, cout = 5 + classes;
    const float eps = 1e-8f;
    for (int b = 0; b < batch; ++b)
        for (int loc = 0; loc < s; ++loc) {
            const float* x = act + (size_t)b * cin * s + loc;
            float side[4];
            for (int sd = 0; sd < 4; ++sd) {
                float mx = -INFINITY;
                for (int k = 0; k < bins; ++k) mx = std::max(mx, finite_or_zero(x[(size_t)(sd * bins + k) * s]));
                float denom = 0.0f, expected = 0.0f;
                for (int k = 0; k < bins; ++k) {
                    const float e = std::exp(std::min(std::max(finite_or_zero(x[(size_t)(sd * bins + k) * s]) - mx, -60.0f), 60.0f));
                    denom += e;
                    expected += (float)k * e;
                }
                side[sd] = expected / std::max(denom, eps);
            }
            const int row = loc / w, col = loc % w;
            const float cx = (float)col + 0.5f, cy = (float)row + 0.5f;
            float left = finite_or_zero((cx - side[0]) / (float)w), top = finite_or_zero((cy - side[1]) / (float)h);
            float right = finite_or_zero((cx + side[2]) / (float)w), bottom = finite_or_zero((cy + side[3]) / (float)h);
            if (right < left) std::swap(left, right);
            if (bottom < top) std::swap(top, bottom);
            float bx = finite_or_zero(0.5f * (left + right)), by = finite_or_zero(0.5f * (top + bottom));
            float bw = std::max(finite_or_zero(std::max(right - left, 1e-6f)), 1e-6f), bh = std::max(finite_or_zero(std::max(bottom - top, 1e-6f)), 1e-6f);
            float* o = out + (size_t)b * cout * s + loc;
            o[0] = bx; o[(size_t)s] = by; o[(size_t)2 * s] = bw; o[(size_t)3 * s] = bh;
            for (int e = 0; e < classes + 1; ++e) o[(size_t)(4 + e) * s] = x[(size_t)(coords + e) * s];
        }
    return 0;
}

// Standalone decode+NMS of one image given raw head tensors.
// meta per head (8 floats): gw, gh, classes, n_anchor, scale_x_y, new_coords, then
// anchors are passed in `anchors` as consecutive (w,h) pairs per head.
int orc_decode_nms(int n_heads, const float* const* heads, const float* meta, const float* anchors, int net_w, int net_h,
                   int img_w, int img_h, float thr, float nms_thr, int letterbox, int top_k, int det_exp, int skip_pass1,
                   float* out, int max_out) {
    ORC_TRY
    std::vector<const float*> hp(heads, heads + n_heads);
    std::vector<HeadSpec> specs(n_heads);
    const float* a = anchors;
    for (int k = 0; k < n_heads; ++k) {
        const float* m = meta + 8 * k;
        specs[k].gw = (int)m[0]; specs[k].gh = (int)m[1]; specs[k].classes = (int)m[2]; specs[k].n_anchor = (int)m[3];
        specs[k].scale_x_y = m[4]; specs[k].new_coords = (int)m[5]; specs[k].kind = (int)m[6];
        specs[k].anchors_wh = a;
        a += 2 * specs[k].n_anchor;
    }
    auto d = detect_image(hp, specs, net_w, net_h, img_w, img_h, thr, nms_thr, letterbox != 0, top_k, det_exp != 0, skip_pass1 != 0);
    for (int i = 0; i < (int)d.size() && i < max_out; ++i) {
        float* r = out + 7 * i;
        r[0] = (float)d[i].class_id; r[1] = d[i].conf; r[2] = d[i].obj; r[3] = d[i].x; r[4] = d[i].y; r[5] = d[i].w; r[6] = d[i].h;
    }
    return (int)d.size();
    ORC_CATCH(-1)
}

// Decode only (no NMS, no sort): candidates in emission order.
int orc_decode_only(int n_heads, const float* const* heads, const float* meta, const float* anchors, int net_w, int net_h,
                    int img_w, int img_h, float thr, int letterbox, int det_exp, float* out, int max_out) {
    ORC_TRY
    std::vector<Det> d;
    const float* a = anchors;
    for (int k = 0; k < n_heads; ++k) {
        const float* m = meta + 8 * k;
        HeadSpec hs;
        hs.gw = (int)m[0]; hs.gh = (int)m[1]; hs.classes = (int)m[2]; hs.n_anchor = (int)m[3];
        hs.scale_x_y = m[4]; hs.new_coords = (int)m[5]; hs.kind = (int)m[6]; hs.anchors_wh = a;
        a += 2 * hs.n_anchor;
        decode_head(heads[k], hs, net_w, net_h, img_w, img_h, thr, letterbox != 0, det_exp != 0, d);
    }
    for (int i = 0; i < (int)d.size() && i < max_out; ++i) {
        float* r = out + 7 * i;
        r[0] = (float)d[i].class_id; r[1] = d[i].conf; r[2] = d[i].obj; r[3] = d[i].x; r[4] = d[i].y; r[5] = d[i].w; r[6] = d[i].h;
    }
    return (int)d.size();
    ORC_CATCH(-1)
}

// NMS passes on caller-supplied records (7 floats each, emission order): the
// sequence of decode_network_detections after decoding.  Returns kept count.
int orc_nms_records(float* recs, int n, float nms_thr, int top_k, int skip_pass1) {
    std::vector<Det> d(n);
    for (int i = 0; i < n; ++i) {
        const float* r = recs + 7 * i;
        d[i] = Det{(int)r[0], r[1], r[2], r[3], r[4], r[5], r[6]};
    }
    if (!skip_pass1) apply_nms(d, 1.0f);
    sort_conf_desc(d);
    apply_nms(d, nms_thr);
    sort_conf_desc(d);
    if (top_k > 0 && (int)d.size() > top_k) d.resize(top_k);
    for (int i = 0; i < (int)d.size(); ++i) {
        float* r = recs + 7 * i;
        r[0] = (float)d[i].class_id; r[1] = d[i].conf; r[2] = d[i].obj; r[3] = d[i].x; r[4] = d[i].y; r[5] = d[i].w; r[6] = d[i].h;
    }
    return (int)d.size();
}

// The sorted-list pass of decode_network_detections (stable sort by confidence, then apply_nms) stopped as soon as
// `k` rows have been kept.  On a confidence-sorted list apply_nms always keeps row i and drops later rows, so the rows
// kept up to any point are final: the result is the first k records of the full pass, at the cost of k row scans
// instead of one per survivor.  This is the work the device path does when it is given max_per_image = k; the
// thr = 1.0 pre-pass on the unsorted list (detect.rs:127-128) is not part of it.
int orc_nms_records_first_k(float* recs, int n, float nms_thr, int k) {
    std::vector<Det> d(n);
    for (int i = 0; i < n; ++i) {
        const float* r = recs + 7 * i;
        d[i] = Det{(int)r[0], r[1], r[2], r[3], r[4], r[5], r[6]};
    }
    sort_conf_desc(d);
    std::vector<char> sup((size_t)n, 0);
    std::vector<Det> kept;
    for (int i = 0; i < n && (int)kept.size() < k; ++i) {
        if (sup[i]) continue;
        if (nms_thr > 0.0f)
            for (int j = i + 1; j < n; ++j) {
                if (sup[j] || d[i].class_id != d[j].class_id) continue;
                // sorted: conf[i] >= conf[j], so row i is the one kept (detect.rs:1463-1467)
                if (bbox_iou(d[i], d[j]) > nms_thr) sup[j] = 1;
            }
        kept.push_back(d[i]);
    }
    for (size_t i = 0; i < kept.size(); ++i) {
        float* r = recs + 7 * i;
        const Det& e = kept[i];
        r[0] = (float)e.class_id; r[1] = e.conf; r[2] = e.obj; r[3] = e.x; r[4] = e.y; r[5] = e.w; r[6] = e.h;
    }
    return (int)kept.size();
}

// The same NMS sequence run class by class.  apply_nms never pairs records of different classes
// (detect.rs:1461), so a stable partition by class followed by the per-class passes keeps exactly the
// records the whole-list passes keep; the final order of the reference is confidence descending with
// ties in emission order (two stable sorts, detect.rs:107 and :242), which is rebuilt here from the
// emission index.  Costs the sum of the squared class sizes instead of the squared total.
int orc_nms_records_by_class(float* recs, int n, float nms_thr, int top_k, int skip_pass1) {
    struct Tagged { Det d; int idx; };
    std::map<int, std::vector<Tagged>> by_class;
    for (int i = 0; i < n; ++i) {
        const float* r = recs + 7 * i;
        by_class[(int)r[0]].push_back(Tagged{Det{(int)r[0], r[1], r[2], r[3], r[4], r[5], r[6]}, i});
    }
    std::vector<Tagged> kept;
    for (auto& kv : by_class) {
        std::vector<Tagged>& v = kv.second;
        // the passes of apply_nms restricted to one class; `order` is compacted and permuted together with the
        // records so that every survivor can be traced back to its emission index
        std::vector<Det> d(v.size());
        for (size_t i = 0; i < v.size(); ++i) d[i] = v[i].d;
        std::vector<int> order(v.size());
        for (size_t i = 0; i < v.size(); ++i) order[i] = (int)i;
        auto run_pass = [&](float thr) {
            if (thr <= 0.0f) return;
            const size_t m = d.size();
            std::vector<char> sup(m, 0);
            for (size_t i = 0; i < m; ++i) {
                if (sup[i]) continue;
                for (size_t j = i + 1; j < m; ++j) {
                    if (sup[j]) continue;
                    size_t keep, drop;
                    if (d[i].conf >= d[j].conf) { keep = i; drop = j; } else { keep = j; drop = i; }
                    if (bbox_iou(d[keep], d[drop]) > thr) sup[drop] = 1;
                }
            }
            size_t k = 0;
            for (size_t i = 0; i < m; ++i) if (!sup[i]) { d[k] = d[i]; order[k] = order[i]; ++k; }
            d.resize(k); order.resize(k);
        };
        auto sort_desc = [&]() {
            auto key = [](float f) { int32_t b; std::memcpy(&b, &f, 4); return b < 0 ? (int32_t)(b ^ 0x7fffffff) : b; };
            std::vector<size_t> perm(d.size());
            for (size_t i = 0; i < perm.size(); ++i) perm[i] = i;
            std::stable_sort(perm.begin(), perm.end(), [&](size_t a, size_t b) { return key(d[a].conf) > key(d[b].conf); });
            std::vector<Det> d2(d.size());
            std::vector<int> o2(d.size());
            for (size_t i = 0; i < perm.size(); ++i) { d2[i] = d[perm[i]]; o2[i] = order[perm[i]]; }
            d.swap(d2); order.swap(o2);
        };
        if (!skip_pass1) run_pass(1.0f);
        sort_desc();
        run_pass(nms_thr);
        for (size_t i = 0; i < d.size(); ++i) kept.push_back(Tagged{d[i], v[order[i]].idx});
    }
    auto key = [](float f) { int32_t b; std::memcpy(&b, &f, 4); return b < 0 ? (int32_t)(b ^ 0x7fffffff) : b; };
    std::sort(kept.begin(), kept.end(), [&](const Tagged& a, const Tagged& b) {
        const int32_t ka = key(a.d.conf), kb = key(b.d.conf);
        return ka != kb ? ka > kb : a.idx < b.idx;
    });
    if (top_k > 0 && (int)kept.size() > top_k) kept.resize(top_k);
    for (size_t i = 0; i < kept.size(); ++i) {
        float* r = recs + 7 * i;
        const Det& d = kept[i].d;
        r[0] = (float)d.class_id; r[1] = d.conf; r[2] = d.obj; r[3] = d.x; r[4] = d.y; r[5] = d.w; r[6] = d.h;
    }
    return (int)kept.size();
}

// Single-layer int8 conv: NCHW int8 in, [F][C][k][k] int8 weights, NCHW int32 accumulators out.
void orc_conv_q8_acc_grouped(const int8_t* x, int B, int C, int H, int W, const int8_t* wq, int F, int k, int sx, int sy, int pad, int groups,
                             int32_t* acc) {
    int OH = conv_dim(H, pad, k, sy), OW = conv_dim(W, pad, k, sx);
    conv_q8_acc(x, B, C, H, W, wq, F, k, sx, sy, pad, OH, OW, acc, groups);
}

void orc_conv_q8_acc(const int8_t* x, int B, int C, int H, int W, const int8_t* wq, int F, int k, int sx, int sy, int pad,
                     int32_t* acc) {
    int OH = conv_dim(H, pad, k, sy), OW = conv_dim(W, pad, k, sx);
    conv_q8_acc(x, B, C, H, W, wq, F, k, sx, sy, pad, OH, OW, acc);
}

// Epilogue of the int8 conv on caller-supplied accumulators (NCHW): f32 activation value and int8.
void orc_q8_epilogue(const int32_t* acc, int B, int F, int plane, const float* mult, const float* bias, int act, float inv_sy,
                     float* out_f32, int8_t* out_q8) {
    for (int b = 0; b < B; ++b)
        for (int f = 0; f < F; ++f)
            for (int p = 0; p < plane; ++p) {
                size_t i = ((size_t)b * F + f) * plane + p;
                float a = det_activate((Act)act, std::fma((float)acc[i], mult[f], bias[f]));
                if (out_f32) out_f32[i] = a;
                if (out_q8) out_q8[i] = quant_i8(a, inv_sy);
            }
}

// The same epilogue over floating-point accumulators with an E4M3 output code.
void orc_f8_epilogue(const float* acc, int B, int F, int plane, const float* mult, const float* bias, int act, float inv_sy,
                     float* out_f32, uint8_t* out_f8) {
    for (int b = 0; b < B; ++b)
        for (int f = 0; f < F; ++f)
            for (int p = 0; p < plane; ++p) {
                size_t i = ((size_t)b * F + f) * plane + p;
                float a = det_activate((Act)act, std::fma(acc[i], mult[f], bias[f]));
                if (out_f32) out_f32[i] = a;
                if (out_f8) out_f8[i] = f32_to_e4m3_fast(a * inv_sy);
            }
}

// Convolution of E4M3 codes accumulated in double (NCHW codes, [F][C][k][k] weight codes); taps outside the image are skipped.
// l1 (optional) receives sum |x||w| per output, the yardstick for accumulation-order tolerances.
void orc_conv_f8_acc(const uint8_t* x, int B, int C, int H, int W, const uint8_t* w, int F, int k, int stride, int pad, double* acc, double* l1) {
    const int OH = conv_dim(H, pad, k, stride), OW = conv_dim(W, pad, k, stride);
    float dec[256];
    for (int c = 0; c < 256; ++c) dec[c] = ((c & 0x7F) == 0x7F) ? 0.0f : e4m3_to_f32((uint8_t)c);
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; ++b)
        for (int f = 0; f < F; ++f)
            for (int oy = 0; oy < OH; ++oy)
                for (int ox = 0; ox < OW; ++ox) {
                    double a = 0.0, l = 0.0;
                    for (int ic = 0; ic < C; ++ic)
                        for (int ky = 0; ky < k; ++ky) {
                            const int yy = oy * stride + ky - pad;
                            if (yy < 0 || yy >= H) continue;
                            for (int kx = 0; kx < k; ++kx) {
                                const int xx = ox * stride + kx - pad;
                                if (xx < 0 || xx >= W) continue;
                                const double p = (double)dec[x[(((size_t)b * C + ic) * H + yy) * W + xx]] * (double)dec[w[(((size_t)f * C + ic) * k + ky) * k + kx]];
                                a += p;
                                l += std::fabs(p);
                            }
                        }
                    const size_t o = (((size_t)b * F + f) * OH + oy) * OW + ox;
                    acc[o] = a;
                    if (l1) l1[o] = l;
                }
}

// ---------------------------------------------------------------------------
// Image pre-processing (lightnet-runtime/src/image.rs): u8 interleaved RGB -> planar f32, Darknet's float resize,
// OpenCV's INTER_LINEAR_EXACT resize, letterbox.  Same operations in the same order as the reference, f32 throughout.
// ---------------------------------------------------------------------------

// image.rs:57-89 from_interleaved_rgb_u8: planar[c][y][x] = byte / 255.0
void orc_image_from_u8(const uint8_t* rgb, int w, int h, float* planar) {
    const size_t plane = (size_t)w * h;
    for (size_t i = 0; i < plane; ++i)
        for (int c = 0; c < 3; ++c) planar[c * plane + i] = (float)rgb[i * 3 + c] / 255.0f;
}

// Rust's `x as usize` for a float: NaN and negatives become 0, values beyond the range saturate (here: to INT_MAX).
static inline int f32_as_index(float v) {
    if (!(v > 0.0f)) return 0;
    if (v >= 2147483520.0f) return 2147483647;
    return (int)v;
}

// image.rs:95-151 resize: align-corners bilinear, horizontal pass into an intermediate plane, then vertical.
// (Resizing to a width or height of 1 from a larger source multiplies 0 by an infinite scale: the reference then produces
// NaN pixels, and so does this restatement.)
void orc_image_resize(const float* src, int sw, int sh, int channels, int w, int h, float* out) {
    if (sw == w && sh == h) { std::memcpy(out, src, (size_t)sw * sh * channels * 4); return; }
    const float w_scale = ((float)sw - 1.0f) / ((float)w - 1.0f);
    const float h_scale = ((float)sh - 1.0f) / ((float)h - 1.0f);
    std::vector<float> part((size_t)w * sh * channels);
    for (int ch = 0; ch < channels; ++ch) {
        for (int y = 0; y < sh; ++y) {
            const float* row = src + ((size_t)ch * sh + y) * sw;
            float* dst = part.data() + ((size_t)ch * sh + y) * w;
            for (int c = 0; c < w; ++c) {
                if (c == w - 1 || sw == 1) dst[c] = row[sw - 1];
                else {
                    const float sx = (float)c * w_scale;
                    const int ix = f32_as_index(sx);
                    const float dx = sx - (float)ix;
                    dst[c] = (1.0f - dx) * row[ix] + dx * row[ix + 1];
                }
            }
        }
        for (int y = 0; y < h; ++y) {
            const float sy = sh == 1 ? 0.0f : (float)y * h_scale;
            const int iy = f32_as_index(sy);
            const float dy = sy - (float)iy;
            const float* row0 = part.data() + ((size_t)ch * sh + iy) * w;
            float* dst = out + ((size_t)ch * h + y) * w;
            for (int x = 0; x < w; ++x) dst[x] = (1.0f - dy) * row0[x];
            if (y == h - 1 || sh == 1) continue;
            const float* row1 = part.data() + ((size_t)ch * sh + iy + 1) * w;
            for (int x = 0; x < w; ++x) dst[x] += dy * row1[x];
        }
    }
}

// image.rs:307-327 exact_coeffs: OpenCV INTER_LINEAR_EXACT taps (x0, x1, c0, c1), c0 + c1 == 256.
static void exact_coeffs(int src, int dst, std::vector<int>& x0s, std::vector<int>& x1s, std::vector<uint32_t>& c0s, std::vector<uint32_t>& c1s) {
    x0s.resize(dst); x1s.resize(dst); c0s.resize(dst); c1s.resize(dst);
    for (int d = 0; d < dst; ++d) {
        const double fsx = ((double)d + 0.5) * (double)src / (double)dst - 0.5;
        double x0 = std::floor(fsx);
        double fx = fsx - x0;
        if (x0 < 0.0) { x0 = 0.0; fx = 0.0; }
        if (x0 >= (double)src - 1.0) { x0 = (double)src - 1.0; fx = 0.0; }
        const int i0 = (int)x0;
        const uint32_t c1 = (uint32_t)std::floor(fx * 256.0 + 0.5);
        x0s[d] = i0; x1s[d] = std::min(i0 + 1, src - 1); c0s[d] = 256 - c1; c1s[d] = c1;
    }
}

// image.rs:157-190 resize_linear_exact on the u8 source: horizontal pass in 1/256, vertical in 1/65536, rounded.
void orc_image_resize_exact_u8(const uint8_t* src, int sw, int sh, int w, int h, uint8_t* out) {
    if (sw == w && sh == h) { std::memcpy(out, src, (size_t)sw * sh * 3); return; }
    std::vector<int> x0, x1, y0, y1;
    std::vector<uint32_t> cx0, cx1, cy0, cy1;
    exact_coeffs(sw, w, x0, x1, cx0, cx1);
    exact_coeffs(sh, h, y0, y1, cy0, cy1);
    std::vector<uint32_t> tmp((size_t)sh * w * 3);
    for (int y = 0; y < sh; ++y)
        for (int x = 0; x < w; ++x)
            for (int ch = 0; ch < 3; ++ch)
                tmp[((size_t)y * w + x) * 3 + ch] = (uint32_t)src[((size_t)y * sw + x0[x]) * 3 + ch] * cx0[x] + (uint32_t)src[((size_t)y * sw + x1[x]) * 3 + ch] * cx1[x];
    for (int y = 0; y < h; ++y)
        for (int i = 0; i < w * 3; ++i) {
            const uint32_t v = tmp[(size_t)y0[y] * w * 3 + i] * cy0[y] + tmp[(size_t)y1[y] * w * 3 + i] * cy1[y];
            out[(size_t)y * w * 3 + i] = (uint8_t)((v + 32768u) >> 16);
        }
}

// image.rs:329-341 fit_inside
void orc_image_fit_inside(int sw, int sh, int dw, int dh, int* nw, int* nh) {
    if (((float)dw / (float)sw) < ((float)dh / (float)sh)) { *nw = std::max(dw, 1); *nh = std::max((int)((long long)sh * dw / sw), 1); }
    else { *nw = std::max((int)((long long)sw * dh / sh), 1); *nh = std::max(dh, 1); }
}

// image.rs:203-229 letterbox: float resize to fit, 0.5 padding, integer offsets (dst - new) / 2.
void orc_image_letterbox(const float* src, int sw, int sh, int channels, int w, int h, float* out) {
    int nw, nh;
    orc_image_fit_inside(sw, sh, w, h, &nw, &nh);
    std::vector<float> resized((size_t)nw * nh * channels);
    orc_image_resize(src, sw, sh, channels, nw, nh, resized.data());
    for (size_t i = 0; i < (size_t)w * h * channels; ++i) out[i] = 0.5f;
    const int xo = (w - nw) / 2, yo = (h - nh) / 2;
    for (int ch = 0; ch < channels; ++ch)
        for (int y = 0; y < nh; ++y)
            std::memcpy(out + ((size_t)ch * h + y + yo) * w + xo, resized.data() + ((size_t)ch * nh + y) * nw, (size_t)nw * 4);
}

// Single f32 conv layer in the reference loop order (folded weights + bias), NCHW.
void orc_conv_f32(const float* x, int B, int C, int H, int W, const float* w, const float* bias, int F, int k, int sx, int sy,
                  int pad, int groups, int act, float* y) {
    Layer L;
    L.filters = F; L.size = k; L.stride_x = sx; L.stride_y = sy; L.padding = pad; L.groups = groups; L.act = (Act)act;
    Shape is; is.w = W; is.h = H; is.c = C; is.b = B;
    Shape os; os.w = conv_dim(W, pad, k, sx); os.h = conv_dim(H, pad, k, sy); os.c = F; os.b = B;
    Tensor xt(is), yt(os);
    std::memcpy(xt.d.data(), x, xt.d.size() * 4);
    std::vector<float> fw(w, w + (size_t)F * (C / std::max(groups, 1)) * k * k), fb(bias, bias + F);
    conv_f32(L, xt, yt, true, &fw, &fb);
    std::memcpy(y, yt.d.data(), yt.d.size() * 4);
}

void orc_maxpool_f32(const float* x, int B, int C, int H, int W, int size, int sx, int sy, int padding, float* y) {
    Layer L;
    L.size = size; L.stride_x = sx; L.stride_y = sy; L.padding = padding;
    Shape is; is.w = W; is.h = H; is.c = C; is.b = B;
    Shape os; os.w = pool_dim(W, padding, size, sx); os.h = pool_dim(H, padding, size, sy); os.c = C; os.b = B;
    Tensor xt(is), yt(os);
    std::memcpy(xt.d.data(), x, xt.d.size() * 4);
    maxpool_f32(L, xt, yt);
    std::memcpy(y, yt.d.data(), yt.d.size() * 4);
}

float orc_activate(int act, float v) { return activate((Act)act, v); }
float orc_det_activate(int act, float v) { return det_activate((Act)act, v); }
float orc_det_expf(float v) { return det_expf(v); }
float orc_bbox_iou(const float* a, const float* b) {
    Det da{0, 0, 0, a[0], a[1], a[2], a[3]}, db{0, 0, 0, b[0], b[1], b[2], b[3]};
    return bbox_iou(da, db);
}
unsigned char orc_f32_to_e4m3(float v) { return f32_to_e4m3(v); }
float orc_e4m3_to_f32(unsigned char b) { return e4m3_to_f32(b); }
int8_t orc_quant_i8(float a, float inv_s) { return quant_i8(a, inv_s); }

}  // extern "C"
