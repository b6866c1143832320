// [yolo] decode + per-class greedy NMS on the device.
//
// Reference semantics (lightnet-train/src/detect.rs): decode_yolo_head (:934-1016) emits one candidate per
// (head, anchor, cell, class) with objectness > thr and confidence = objectness * class_prob > thr, in that
// order; the list is stably sorted by confidence descending (:107) and apply_nms (:1449-1484) walks it: a
// candidate survives unless an earlier survivor of the same class overlaps it with IoU > nms_thr.
//
// Device formulation.  Every candidate gets the 64-bit key (order-preserving confidence bits << 32) |
// ~emission_index; descending key order is exactly the reference's sorted order, ties included.  Greedy NMS
// only ever needs candidates in that order, and only until top_k survivors exist, so the candidates are
// consumed in bands from the top: a radix selection over the key (12-bit digits, histogram in shared memory,
// descending only into a digit that holds too many candidates) finds a cut such that the band above it fits
// in shared memory; the band is collected, sorted (bitonic) and resolved by one CTA per image: each 512-
// candidate chunk is tested against the survivors so far, a 512 x 512 same-class IoU bitmask is built, and
// one warp resolves it with ballot/shuffle.  Images stop as soon as they have top_k survivors or run out of
// candidates.  The head tensors are the only large input; they are re-read once per selection / collection
// pass and nothing of candidate size is ever written to HBM.
//
// All arithmetic that decides an ordering or a threshold (sigmoid, box decode, IoU) uses single IEEE-754
// operations in the reference's evaluation order, so a CPU evaluating the same expressions gets the same bits.
#include <cstdlib>
#include <ctime>

#include "ln_conv_plan.h"

namespace {

constexpr int kMaxHeads = 8;
constexpr int kBandMaxLarge = 16384;  // candidates of one band (sorted in shared memory) when at most 1024 survivors are wanted
constexpr int kBandMaxSmall = 8192;   // ... when more are wanted (their boxes need the room)
constexpr int kChunk = 512;      // candidates resolved per bitmask step
constexpr int kBins = 4096;      // 12-bit radix digits
constexpr unsigned kFlatChunk = 32768;  // cached score keys one block of the flat passes walks
constexpr int kLevels = 6;       // 5 x 12 bits + 4 bits = 64

enum { PHASE_SELECT = 0, PHASE_BAND = 1, PHASE_DONE = 2 };

struct HeadDev {
    const float* raw;  // [batch][n_anchor*(5+classes)][gh*gw]
    int gw, gh, classes, n_anchor, new_coords;
    float scale_x_y;
    float anchors[16];
    int ca_base;  // number of (anchor, cell) slots in earlier heads
};

struct YoloParams {
    HeadDev heads[kMaxHeads];
    int n_heads, batch, total_ca, classes;
    int net_w, net_h, letterbox;
    float thr, nms_thr;
    int k_eff;          // survivors wanted per image
    int max_per_image;  // record capacity
    int band_max;       // capacity of one band
    unsigned cache_stride;  // cached score keys per image (total_ca * classes rounded up to 4)
};

struct ImgState {
    unsigned long long hi;      // keys >= hi have been consumed
    unsigned long long lo;      // current band is [lo, hi)
    unsigned long long prefix;  // digits fixed so far by the radix selection
    int level, phase, cap, above, band_count, kept, exhausted, img_w, img_h, last_gain;  // last_gain: survivors the previous band added
};

__device__ __forceinline__ int level_shift(int l) { return l < 5 ? 52 - 12 * l : 0; }
__device__ __forceinline__ int level_bits(int l) { return l < 5 ? 12 : 4; }

__device__ __forceinline__ float head_act(float raw, int new_coords) { return new_coords ? raw : ln_det_sigmoid(raw); }

__device__ __forceinline__ unsigned conf_key(float c) {
    unsigned b = __float_as_uint(c);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_conf(unsigned k) {
    unsigned b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
    return __uint_as_float(b);
}

struct Box { float x, y, w, h; };

// detect.rs:1288-1322 decode_bbox followed by :1414-1447 correct_bbox, operation for operation.
__device__ __forceinline__ Box decode_box(const HeadDev& h, const float* img, int a, int idx, int net_w, int net_h, int img_w, int img_h,
                                          int letterbox) {
    const int stride = h.gw * h.gh, epa = h.classes + 5;
    const int row = idx / h.gw, col = idx - row * h.gw;
    const float tx = img[(size_t)(a * epa + 0) * stride + idx], ty = img[(size_t)(a * epa + 1) * stride + idx];
    const float tw = img[(size_t)(a * epa + 2) * stride + idx], th = img[(size_t)(a * epa + 3) * stride + idx];
    const float s = h.scale_x_y, nw = (float)net_w, nh = (float)net_h, iw = (float)img_w, ih = (float)img_h;
    const float half = __fmul_rn(0.5f, __fsub_rn(s, 1.0f));
    float bx = __fdiv_rn(__fsub_rn(__fadd_rn((float)col, __fmul_rn(s, head_act(tx, h.new_coords))), half), (float)h.gw);
    float by = __fdiv_rn(__fsub_rn(__fadd_rn((float)row, __fmul_rn(s, head_act(ty, h.new_coords))), half), (float)h.gh);
    float bw, bh;
    const float aw = h.anchors[2 * a], ah = h.anchors[2 * a + 1];
    if (h.new_coords) {
        bw = __fdiv_rn(__fmul_rn(__fmul_rn(__fmul_rn(tw, tw), 4.0f), aw), nw);
        bh = __fdiv_rn(__fmul_rn(__fmul_rn(__fmul_rn(th, th), 4.0f), ah), nh);
    } else {
        bw = __fdiv_rn(__fmul_rn(ln_det_expf(tw), aw), nw);
        bh = __fdiv_rn(__fmul_rn(ln_det_expf(th), ah), nh);
    }
    float new_w, new_h;
    if (letterbox) {
        if (__fdiv_rn(nw, iw) < __fdiv_rn(nh, ih)) { new_w = nw; new_h = __fdiv_rn(__fmul_rn(ih, nw), iw); }
        else { new_w = __fdiv_rn(__fmul_rn(iw, nh), ih); new_h = nh; }
    } else { new_w = nw; new_h = nh; }
    const float delta_w = __fsub_rn(nw, new_w), delta_h = __fsub_rn(nh, new_h);
    const float ratio_w = __fdiv_rn(new_w, nw), ratio_h = __fdiv_rn(new_h, nh);
    bx = __fdiv_rn(__fsub_rn(bx, __fdiv_rn(__fdiv_rn(delta_w, 2.0f), nw)), ratio_w);
    by = __fdiv_rn(__fsub_rn(by, __fdiv_rn(__fdiv_rn(delta_h, 2.0f), nh)), ratio_h);
    bw = __fdiv_rn(bw, ratio_w);
    bh = __fdiv_rn(bh, ratio_h);
    Box b;
    b.x = __fmul_rn(bx, iw); b.y = __fmul_rn(by, ih); b.w = __fmul_rn(bw, iw); b.h = __fmul_rn(bh, ih);
    return b;
}

// detect.rs:1486-1503 bbox_iou with detection_geometry.rs:14-30 edges
__device__ __forceinline__ float box_iou(const Box& a, const Box& b) {
    const float al = __fsub_rn(a.x, __fmul_rn(a.w, 0.5f)), at = __fsub_rn(a.y, __fmul_rn(a.h, 0.5f));
    const float ar = __fadd_rn(a.x, __fmul_rn(a.w, 0.5f)), ab = __fadd_rn(a.y, __fmul_rn(a.h, 0.5f));
    const float bl = __fsub_rn(b.x, __fmul_rn(b.w, 0.5f)), bt = __fsub_rn(b.y, __fmul_rn(b.h, 0.5f));
    const float br = __fadd_rn(b.x, __fmul_rn(b.w, 0.5f)), bb = __fadd_rn(b.y, __fmul_rn(b.h, 0.5f));
    const float iw = fmaxf(__fsub_rn(fminf(ar, br), fmaxf(al, bl)), 0.0f), ih = fmaxf(__fsub_rn(fminf(ab, bb), fmaxf(at, bt)), 0.0f);
    const float inter = __fmul_rn(iw, ih);
    if (inter <= 0.0f) return 0.0f;
    const float aa = __fmul_rn(fmaxf(a.w, 0.0f), fmaxf(a.h, 0.0f)), ba = __fmul_rn(fmaxf(b.w, 0.0f), fmaxf(b.h, 0.0f));
    return __fdiv_rn(inter, __fsub_rn(__fadd_rn(aa, ba), inter));
}

__device__ __forceinline__ int find_head(const YoloParams& p, int ca) {
    int h = 0;
    for (int k = 1; k < p.n_heads; ++k)
        if (ca >= p.heads[k].ca_base) h = k;
    return h;
}

// One pass over the candidates.  MODE 0: histogram of the current radix digit of the still unconsumed candidates.
// MODE 1: collect the keys of the band [lo, hi).  One thread per (anchor, cell); blockIdx.y = image.
// FIRST: read the head tensors, evaluate the scores and leave their 32-bit order-preserving keys (0 = not a
// candidate) in `cache`, laid out [image][class][anchor-cell]; later passes read the cache instead and do
// integer work only.
template <int MODE, bool FIRST>
__global__ void __launch_bounds__(256) yolo_scan_kernel(const __grid_constant__ YoloParams p, ImgState* __restrict__ states,
                                                        unsigned* __restrict__ hist, unsigned long long* __restrict__ band,
                                                        int* __restrict__ band_fill, unsigned* __restrict__ cache) {
    const int img = blockIdx.y;
    const ImgState st = states[img];
    if (!FIRST && (MODE == 0 ? st.phase != PHASE_SELECT : st.phase != PHASE_BAND)) return;
    __shared__ unsigned s_hist[MODE == 0 ? kBins : 1];
    if (MODE == 0) {
        for (int i = threadIdx.x; i < kBins; i += blockDim.x) s_hist[i] = 0;
        __syncthreads();
    }
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    const int ca = blockIdx.x * blockDim.x + threadIdx.x;
    if (ca < p.total_ca) {
        unsigned* img_cache = cache + (size_t)img * p.cache_stride;
        const float* img_raw = nullptr;
        int stride = 0, a = 0, idx = 0, epa = 0, new_coords = 0;
        float obj = 0.0f;
        if (FIRST) {
            const HeadDev& h = p.heads[find_head(p, ca)];
            stride = h.gw * h.gh; epa = h.classes + 5; new_coords = h.new_coords;
            const int local = ca - h.ca_base;
            a = local / stride; idx = local - a * stride;
            img_raw = h.raw + (size_t)img * h.n_anchor * epa * stride;
            obj = head_act(img_raw[(size_t)(a * epa + 4) * stride + idx], new_coords);
        }
        // consecutive classes often fall into the same bin (always, when scores saturate): count runs in registers
        unsigned run_bin = 0xFFFFFFFFu, run_len = 0;
        for (int c = 0; c < p.classes; ++c) {
            unsigned ck;
            if (FIRST) {
                ck = 0;
                if (obj > p.thr) {
                    const float conf = __fmul_rn(obj, head_act(img_raw[(size_t)(a * epa + 5 + c) * stride + idx], new_coords));
                    if (conf > p.thr) ck = conf_key(conf);
                }
                img_cache[(size_t)c * p.total_ca + ca] = ck;
            } else {
                ck = img_cache[(size_t)c * p.total_ca + ca];
            }
            if (ck == 0u) continue;
            const unsigned eidx = (unsigned)ca * (unsigned)p.classes + (unsigned)c;
            const unsigned long long key = ((unsigned long long)ck << 32) | (unsigned long long)(0xFFFFFFFFu - eidx);
            if (key >= st.hi) continue;
            if (MODE == 0) {
                if (st.level > 0 && (key >> (shift + bits)) != st.prefix) continue;
                const unsigned bin = (unsigned)(key >> shift) & ((1u << bits) - 1u);
                if (bin == run_bin) ++run_len;
                else {
                    if (run_len) atomicAdd(&s_hist[run_bin], run_len);
                    run_bin = bin;
                    run_len = 1;
                }
            } else {
                if (key < st.lo) continue;
                const int slot = atomicAdd(&band_fill[img], 1);
                if (slot < p.band_max) band[(size_t)img * p.band_max + slot] = key;
            }
        }
        if (MODE == 0 && run_len) atomicAdd(&s_hist[run_bin], run_len);
    }
    if (MODE == 0) {
        __syncthreads();
        for (int i = threadIdx.x; i < kBins; i += blockDim.x)
            if (s_hist[i]) atomicAdd(&hist[(size_t)img * kBins + i], s_hist[i]);
    }
}

// Later passes: one thread per cached score key (flat over [class][anchor-cell]); integer work only.  Lanes of a warp
// that fall into the same histogram bin (all of them, when scores saturate) are merged into one shared-memory add.
template <int MODE>
__global__ void __launch_bounds__(256) yolo_scan_cached_kernel(const __grid_constant__ YoloParams p, const ImgState* __restrict__ states,
                                                               unsigned* __restrict__ hist, unsigned long long* __restrict__ band,
                                                               int* __restrict__ band_fill, const unsigned* __restrict__ cache) {
    const int img = blockIdx.y;
    const ImgState st = states[img];
    if (MODE == 0 ? st.phase != PHASE_SELECT : st.phase != PHASE_BAND) return;
    __shared__ unsigned s_hist[MODE == 0 ? kBins : 1];
    if (MODE == 0) {
        for (int i = threadIdx.x; i < kBins; i += blockDim.x) s_hist[i] = 0;
        __syncthreads();
    }
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    const unsigned per_image = (unsigned)p.total_ca * (unsigned)p.classes;
    const unsigned chunk_begin = blockIdx.x * kFlatChunk;
    const unsigned* img_cache = cache + (size_t)img * p.cache_stride;
    // four keys per thread per step (one 16-byte load); the trip count is uniform over the block
    for (unsigned base = chunk_begin; base < chunk_begin + kFlatChunk && base < per_image; base += 4u * blockDim.x) {
        const unsigned i0 = base + 4u * threadIdx.x;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (i0 < per_image) v = *reinterpret_cast<const uint4*>(img_cache + i0);  // the padding of the last vector is zero
        const unsigned cks[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const unsigned i = i0 + e, ck = cks[e];
            bool valid = false;
            unsigned bin = 0xFFFFFFFFu;
            unsigned long long key = 0;
            if (ck != 0u) {
                const unsigned c = i / (unsigned)p.total_ca, ca = i - c * (unsigned)p.total_ca;
                const unsigned eidx = ca * (unsigned)p.classes + c;
                key = ((unsigned long long)ck << 32) | (unsigned long long)(0xFFFFFFFFu - eidx);
                valid = key < st.hi;
                if (MODE == 0) valid = valid && (st.level == 0 || (key >> (shift + bits)) == st.prefix);
                else valid = valid && key >= st.lo;
            }
            if (MODE == 0) {
                if (valid) bin = (unsigned)(key >> shift) & ((1u << bits) - 1u);
                const unsigned same = __match_any_sync(0xffffffffu, bin);
                if (valid && (threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&s_hist[bin], (unsigned)__popc(same));
            } else if (valid) {
                const int slot = atomicAdd(&band_fill[img], 1);
                if (slot < p.band_max) band[(size_t)img * p.band_max + slot] = key;
            }
        }
    }
    if (MODE == 0) {
        __syncthreads();
        for (int b = threadIdx.x; b < kBins; b += blockDim.x)
            if (s_hist[b]) atomicAdd(&hist[(size_t)img * kBins + b], s_hist[b]);
    }
}

// One block per image: walk the digit histogram from the top, either fix the band's lower bound or descend
// into the digit that holds too many candidates.  Leaves the histogram zeroed.
__global__ void __launch_bounds__(256) yolo_select_kernel(const __grid_constant__ YoloParams p, ImgState* __restrict__ states,
                                                          unsigned* __restrict__ hist, int* __restrict__ pending) {
    const int img = blockIdx.x;
    ImgState st = states[img];
    if (st.phase != PHASE_SELECT) return;
    __shared__ unsigned s_part[256];
    __shared__ unsigned s_h[kBins];
    unsigned* h = hist + (size_t)img * kBins;
    const int nb = 1 << level_bits(st.level);
    const int per = kBins / 256;  // 16 bins per thread; thread t owns, from the top, bins nb-1-16t .. nb-1-16t-15
    unsigned sum = 0;
    for (int j = 0; j < per; ++j) {
        const int slot = threadIdx.x * per + j;  // slot 0 = top bin
        const int bin = nb - 1 - slot;
        const unsigned v = bin >= 0 ? h[bin] : 0u;
        s_h[slot] = v;
        sum += v;
        if (bin >= 0) h[bin] = 0u;
    }
    s_part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x != 0) return;
    // ---- one thread decides (a few hundred steps at most)
    if (st.level == 0) {
        // band size: four candidates per survivor still wanted, or more when the previous band showed heavier suppression
        long long want = 4ll * (p.k_eff - st.kept);
        if (st.last_gain >= 0) {
            const long long per = ((long long)st.band_count * 3 / 2) / (st.last_gain > 0 ? st.last_gain : 1) + 1;
            if (per > 4) want = per * (p.k_eff - st.kept);
        }
        st.cap = want < 1024 ? 1024 : (want > p.band_max ? p.band_max : (int)want);
        st.above = 0;
        st.prefix = 0;
    }
    const unsigned cap_left = (unsigned)(st.cap - st.above);
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    unsigned cum = 0;
    int owner = -1;
    for (int t = 0; t < 256; ++t) {
        if (cum + s_part[t] > cap_left) { owner = t; break; }
        cum += s_part[t];
    }
    if (owner < 0) {
        // everything that is left (under this prefix) fits into the band
        st.lo = st.level == 0 ? 0ull : (st.prefix << (shift + bits));
        st.band_count = st.above + (int)cum;
        st.exhausted = st.level == 0 ? 1 : 0;
        st.phase = PHASE_BAND;
        states[img] = st;
        return;
    }
    int b = -1;
    for (int j = 0; j < per; ++j) {
        const int slot = owner * per + j;
        if (cum + s_h[slot] > cap_left) { b = nb - 1 - slot; break; }
        cum += s_h[slot];
    }
    const int total = st.above + (int)cum;
    const bool last = st.level == kLevels - 1;
    if (total >= st.cap / 4 || last) {
        const unsigned long long base = st.level == 0 ? 0ull : (st.prefix << (shift + bits));
        st.lo = base + ((unsigned long long)(b + 1) << shift);  // b+1 == nb carries into the digit above: the band is `above` only
        st.band_count = total;
        st.exhausted = 0;
        st.phase = PHASE_BAND;
    } else {
        st.above = total;
        st.prefix = (st.level == 0 ? 0ull : (st.prefix << bits)) | (unsigned long long)b;
        st.level += 1;
        atomicAdd(pending, 1);
    }
    states[img] = st;
}

__device__ __forceinline__ void bitonic_sort_desc(unsigned long long* keys, int n_pow2) {
    for (int k = 2; k <= n_pow2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n_pow2; i += blockDim.x) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = keys[i], b = keys[ixj];
                    const bool desc = (i & k) == 0;
                    if (desc ? a < b : a > b) { keys[i] = b; keys[ixj] = a; }
                }
            }
            __syncthreads();
        }
    }
}

// One CTA per image: sort the band, then greedy per-class NMS chunk by chunk.
__global__ void __launch_bounds__(1024, 1) yolo_nms_kernel(const __grid_constant__ YoloParams p, ImgState* __restrict__ states,
                                                           const unsigned long long* __restrict__ band, int* __restrict__ band_fill,
                                                           float4* __restrict__ kept_box, int* __restrict__ kept_cls,
                                                           ln_detection* __restrict__ records, int* __restrict__ active) {
    extern __shared__ unsigned char smem[];
    const int img = blockIdx.x;
    ImgState st = states[img];
    if (st.phase != PHASE_BAND) return;
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem);             // band_max
    float4* kbox = reinterpret_cast<float4*>(keys + p.band_max);                          // k_eff survivors
    float4* cbox = kbox + p.k_eff;                                                       // kChunk
    unsigned* mask = reinterpret_cast<unsigned*>(cbox + kChunk);                         // kChunk x 16 words
    int* kcls = reinterpret_cast<int*>(mask + kChunk * (kChunk / 32));                   // k_eff
    int* ccls = kcls + p.k_eff;                                                          // kChunk
    float* cobj = reinterpret_cast<float*>(ccls + kChunk);                               // kChunk
    int* cpos = reinterpret_cast<int*>(cobj + kChunk);                                   // kChunk: survivor slot or -1
    unsigned* alive_words = reinterpret_cast<unsigned*>(cpos + kChunk);                  // 16
    __shared__ int s_kept;

    int n = band_fill[img];
    if (n > p.band_max) n = p.band_max;
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    for (int i = threadIdx.x; i < n2; i += blockDim.x) keys[i] = i < n ? band[(size_t)img * p.band_max + i] : 0ull;
    for (int i = threadIdx.x; i < st.kept; i += blockDim.x) {
        kbox[i] = kept_box[(size_t)img * p.k_eff + i];
        kcls[i] = kept_cls[(size_t)img * p.k_eff + i];
    }
    if (threadIdx.x == 0) s_kept = st.kept;
    __syncthreads();
    bitonic_sort_desc(keys, n2);

    for (int base = 0; base < n; base += kChunk) {
        const int m = min(kChunk, n - base);
        const int kept_before = s_kept;
        // ---- decode the chunk and test it against the survivors so far
        bool alive = false;
        if ((int)threadIdx.x < m) {
            const unsigned long long key = keys[base + threadIdx.x];
            const unsigned eidx = 0xFFFFFFFFu - (unsigned)(key & 0xFFFFFFFFull);
            const int cls = (int)(eidx % (unsigned)p.classes), ca = (int)(eidx / (unsigned)p.classes);
            const int hd = find_head(p, ca);
            const HeadDev& h = p.heads[hd];
            const int stride = h.gw * h.gh, epa = h.classes + 5;
            const int local = ca - h.ca_base, a = local / stride, idx = local - a * stride;
            const float* img_raw = h.raw + (size_t)img * h.n_anchor * epa * stride;
            const Box b = decode_box(h, img_raw, a, idx, p.net_w, p.net_h, st.img_w, st.img_h, p.letterbox);
            cbox[threadIdx.x] = make_float4(b.x, b.y, b.w, b.h);
            ccls[threadIdx.x] = cls;
            cobj[threadIdx.x] = head_act(img_raw[(size_t)(a * epa + 4) * stride + idx], h.new_coords);
            alive = true;
            for (int k = 0; k < kept_before; ++k) {
                if (kcls[k] != cls) continue;
                const float4 kb = kbox[k];
                Box q; q.x = kb.x; q.y = kb.y; q.w = kb.z; q.h = kb.w;
                if (box_iou(q, b) > p.nms_thr) { alive = false; break; }
            }
        }
        if (threadIdx.x < kChunk) {
            const unsigned bal = __ballot_sync(0xffffffffu, alive);
            if ((threadIdx.x & 31) == 0) alive_words[threadIdx.x >> 5] = bal;
            cpos[threadIdx.x] = -1;
        }
        __syncthreads();
        // ---- same-class IoU bitmask: bit j of row i set when j > i suppresses under i
        for (int item = threadIdx.x; item < kChunk * (kChunk / 32); item += blockDim.x) {
            const int i = item >> 4, wd = item & 15;
            unsigned bitsv = 0;
            if (i < m && ((alive_words[i >> 5] >> (i & 31)) & 1u) && (wd << 5) + 31 > i) {
                const float4 bi4 = cbox[i];
                Box bi; bi.x = bi4.x; bi.y = bi4.y; bi.w = bi4.z; bi.h = bi4.w;
                const int ci = ccls[i];
                for (int jj = 0; jj < 32; ++jj) {
                    const int j = (wd << 5) + jj;
                    if (j <= i || j >= m || ccls[j] != ci) continue;
                    const float4 bj4 = cbox[j];
                    Box bj; bj.x = bj4.x; bj.y = bj4.y; bj.w = bj4.z; bj.h = bj4.w;
                    if (box_iou(bi, bj) > p.nms_thr) bitsv |= 1u << jj;
                }
            }
            mask[item] = bitsv;
        }
        __syncthreads();
        // ---- one warp resolves the chunk in order
        if (threadIdx.x < 32) {
            const int lane = threadIdx.x;
            unsigned removed = lane < 16 ? ~alive_words[lane] : 0xFFFFFFFFu;
            int kept_now = kept_before;
            for (int i = 0; i < m && kept_now < p.k_eff; ++i) {
                const unsigned r = __shfl_sync(0xffffffffu, removed, i >> 5);
                if ((r >> (i & 31)) & 1u) continue;
                if (lane < 16) removed |= mask[i * 16 + lane];
                if (lane == 0) cpos[i] = kept_now;
                ++kept_now;
            }
            if (lane == 0) s_kept = kept_now;
        }
        __syncthreads();
        // ---- append the new survivors
        if ((int)threadIdx.x < m && cpos[threadIdx.x] >= 0) {
            const int pos = cpos[threadIdx.x];
            kbox[pos] = cbox[threadIdx.x];
            kcls[pos] = ccls[threadIdx.x];
            kept_box[(size_t)img * p.k_eff + pos] = cbox[threadIdx.x];
            kept_cls[(size_t)img * p.k_eff + pos] = ccls[threadIdx.x];
            if (pos < p.max_per_image) {
                const unsigned long long key = keys[base + threadIdx.x];
                ln_detection d;
                d.class_id = (float)ccls[threadIdx.x];
                d.confidence = key_conf((unsigned)(key >> 32));
                d.objectness = cobj[threadIdx.x];
                const float4 b = cbox[threadIdx.x];
                d.x = b.x; d.y = b.y; d.w = b.z; d.h = b.w;
                records[(size_t)img * p.max_per_image + pos] = d;
            }
        }
        __syncthreads();
        if (s_kept >= p.k_eff) break;
    }
    if (threadIdx.x == 0) {
        st.last_gain = s_kept - st.kept;
        st.band_count = n;
        st.kept = s_kept;
        st.hi = st.lo;
        band_fill[img] = 0;
        if (st.exhausted || st.kept >= p.k_eff) st.phase = PHASE_DONE;
        else {
            st.phase = PHASE_SELECT;
            st.level = 0;
            atomicAdd(active, 1);
        }
        states[img] = st;
    }
}

__global__ void yolo_init_states_kernel(ImgState* states, const int* img_w, const int* img_h, int batch) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch) return;
    ImgState s;
    s.hi = ~0ull; s.lo = 0; s.prefix = 0;
    s.level = 0; s.phase = PHASE_SELECT; s.cap = 0; s.above = 0; s.band_count = 0; s.kept = 0; s.exhausted = 0;
    s.img_w = img_w[i]; s.img_h = img_h[i]; s.last_gain = -1;
    states[i] = s;
}

__global__ void yolo_counts_kernel(const ImgState* states, int* counts, int batch, int max_per_image) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < batch) counts[i] = states[i].kept < max_per_image ? states[i].kept : max_per_image;
}

// ---- decode only (parity helper): per (anchor, cell) counts, then ordered writes ---------------
__global__ void yolo_decode_count_kernel(const __grid_constant__ YoloParams p, int img, int* __restrict__ counts) {
    const int ca = blockIdx.x * blockDim.x + threadIdx.x;
    if (ca >= p.total_ca) return;
    const HeadDev& h = p.heads[find_head(p, ca)];
    const int stride = h.gw * h.gh, epa = h.classes + 5;
    const int local = ca - h.ca_base, a = local / stride, idx = local - a * stride;
    const float* img_raw = h.raw + (size_t)img * h.n_anchor * epa * stride;
    const float obj = head_act(img_raw[(size_t)(a * epa + 4) * stride + idx], h.new_coords);
    int n = 0;
    if (obj > p.thr)
        for (int c = 0; c < h.classes; ++c)
            if (__fmul_rn(obj, head_act(img_raw[(size_t)(a * epa + 5 + c) * stride + idx], h.new_coords)) > p.thr) ++n;
    counts[ca] = n;
}
__global__ void yolo_decode_write_kernel(const __grid_constant__ YoloParams p, int img, int img_w, int img_h, const long long* __restrict__ offsets,
                                         ln_detection* __restrict__ out, long long capacity) {
    const int ca = blockIdx.x * blockDim.x + threadIdx.x;
    if (ca >= p.total_ca) return;
    const HeadDev& h = p.heads[find_head(p, ca)];
    const int stride = h.gw * h.gh, epa = h.classes + 5;
    const int local = ca - h.ca_base, a = local / stride, idx = local - a * stride;
    const float* img_raw = h.raw + (size_t)img * h.n_anchor * epa * stride;
    const float obj = head_act(img_raw[(size_t)(a * epa + 4) * stride + idx], h.new_coords);
    if (!(obj > p.thr)) return;
    long long o = offsets[ca];
    Box b;
    bool have = false;
    for (int c = 0; c < h.classes; ++c) {
        const float conf = __fmul_rn(obj, head_act(img_raw[(size_t)(a * epa + 5 + c) * stride + idx], h.new_coords));
        if (!(conf > p.thr)) continue;
        if (!have) { b = decode_box(h, img_raw, a, idx, p.net_w, p.net_h, img_w, img_h, p.letterbox); have = true; }
        if (o < capacity) {
            ln_detection d;
            d.class_id = (float)c; d.confidence = conf; d.objectness = obj; d.x = b.x; d.y = b.y; d.w = b.w; d.h = b.h;
            out[o] = d;
        }
        ++o;
    }
}

int fill_params(ln_ctx* ctx, YoloParams* p, const ln_yolo_head* heads, int32_t n_heads, int32_t net_w, int32_t net_h, const char* who) {
    if (n_heads < 1 || n_heads > kMaxHeads) return ln_fail(ctx, LN_ERR_ARG, "%s: between 1 and %d heads are supported", who, kMaxHeads);
    memset(p, 0, sizeof *p);
    p->n_heads = n_heads; p->net_w = net_w; p->net_h = net_h;
    int ca = 0;
    for (int k = 0; k < n_heads; ++k) {
        const ln_yolo_head& s = heads[k];
        if (!s.raw || s.raw->dtype != LN_F32) return ln_fail(ctx, LN_ERR_ARG, "%s: head %d is not an f32 tensor", who, k);
        if (s.n_anchor < 1 || s.n_anchor > 8 || s.classes < 1) return ln_fail(ctx, LN_ERR_ARG, "%s: head %d has %d anchors / %d classes", who, k, s.n_anchor, s.classes);
        // decode_yolo_head's length check (detect.rs:950-959)
        if (s.raw->c != (int64_t)s.n_anchor * (s.classes + 5)) return ln_fail(ctx, LN_ERR_SHAPE, "YOLO head tensor length mismatch: head %d has %lld channels, expected %d", k, (long long)s.raw->c, s.n_anchor * (s.classes + 5));
        if (k > 0 && (s.raw->n != heads[0].raw->n || s.classes != heads[0].classes)) return ln_fail(ctx, LN_ERR_SHAPE, "%s: heads disagree on batch or class count", who);
        HeadDev& h = p->heads[k];
        h.raw = (const float*)s.raw->ptr;
        h.gw = (int)s.raw->w; h.gh = (int)s.raw->h; h.classes = s.classes; h.n_anchor = s.n_anchor; h.new_coords = s.new_coords;
        h.scale_x_y = s.scale_x_y;
        for (int i = 0; i < 2 * s.n_anchor; ++i) h.anchors[i] = s.anchors[i];
        h.ca_base = ca;
        ca += s.n_anchor * h.gw * h.gh;
    }
    p->total_ca = ca;
    p->classes = heads[0].classes;
    p->batch = (int)heads[0].raw->n;
    if ((int64_t)ca * p->classes >= 0xFFFFFFFFll) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "%s: more than 2^32 candidates per image", who);
    return LN_OK;
}

}  // namespace

extern "C" {

int32_t ln_yolo_decode_nms(ln_ctx* ctx, const ln_yolo_head* heads, int32_t n_heads, int32_t net_w, int32_t net_h, const int32_t* image_w,
                           const int32_t* image_h, const ln_detect_options* opts, ln_detection* records_host, int32_t* counts_host) {
    if (!ctx || !heads || !image_w || !image_h || !opts || !records_host || !counts_host) return ln_fail(ctx, LN_ERR_ARG, "ln_yolo_decode_nms: NULL argument");
    if (opts->max_per_image < 1) return ln_fail(ctx, LN_ERR_ARG, "ln_yolo_decode_nms: max_per_image must be positive");
    YoloParams p;
    int rc = fill_params(ctx, &p, heads, n_heads, net_w, net_h, "ln_yolo_decode_nms");
    if (rc) return rc;
    p.thr = opts->confidence_threshold;
    p.nms_thr = opts->nms_threshold;
    p.letterbox = opts->letterbox;
    p.max_per_image = opts->max_per_image;
    p.k_eff = opts->top_k > 0 && opts->top_k < opts->max_per_image ? opts->top_k : opts->max_per_image;
    p.band_max = p.k_eff <= 1024 ? kBandMaxLarge : kBandMaxSmall;
    if (p.k_eff > 4096) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "ln_yolo_decode_nms: at most 4096 detections per image (top_k / max_per_image)");
    for (int i = 0; i < p.batch; ++i)
        if (image_w[i] <= 0 || image_h[i] <= 0) return ln_fail(ctx, LN_ERR_ARG, "image dimensions must be positive for network detection decoding");
    cudaSetDevice(ctx->device);
    const int B = p.batch;
    // scratch: states | hist | band | band_fill | kept | records | sizes | flags
    const size_t sz_states = (size_t)ln_round_up((int64_t)B * sizeof(ImgState), 256);
    const size_t sz_hist = (size_t)B * kBins * 4;
    const size_t sz_band = (size_t)B * p.band_max * 8;
    const size_t sz_fill = (size_t)ln_round_up((int64_t)B * 4, 256);
    const size_t sz_kbox = (size_t)B * p.k_eff * sizeof(float4);
    const size_t sz_kcls = (size_t)ln_round_up((int64_t)B * p.k_eff * 4, 256);
    const size_t sz_rec = (size_t)ln_round_up((int64_t)B * p.max_per_image * sizeof(ln_detection), 256);
    const size_t sz_dims = (size_t)ln_round_up((int64_t)B * 8, 256);
    const size_t sz_cnt = (size_t)ln_round_up((int64_t)B * 4, 256);
    p.cache_stride = (unsigned)ln_round_up((int64_t)p.total_ca * p.classes, 4);
    const size_t sz_cache = (size_t)ln_round_up((int64_t)B * p.cache_stride * 4, 256);  // score keys of every (cell, anchor, class)
    const size_t total = sz_states + sz_hist + sz_band + sz_fill + sz_kbox + sz_kcls + sz_rec + sz_dims + sz_cnt + sz_cache + 256;
    unsigned char* scratch = (unsigned char*)ln_pool_alloc(ctx, total);
    if (!scratch) return LN_ERR_CUDA;
    unsigned char* q = scratch;
    ImgState* states = (ImgState*)q; q += sz_states;
    unsigned* hist = (unsigned*)q; q += sz_hist;
    unsigned long long* band = (unsigned long long*)q; q += sz_band;
    int* band_fill = (int*)q; q += sz_fill;
    float4* kept_box = (float4*)q; q += sz_kbox;
    int* kept_cls = (int*)q; q += sz_kcls;
    ln_detection* records = (ln_detection*)q; q += sz_rec;
    int* dims = (int*)q; q += sz_dims;
    int* counts = (int*)q; q += sz_cnt;
    unsigned* cache = (unsigned*)q; q += sz_cache;
    int* flags = (int*)q;  // [0] pending selections, [1] images still active

    auto fail = [&](int code) { ln_pool_free(ctx, scratch, total); return code; };
#define LN_Y(call)                                                                                            \
    do {                                                                                                      \
        cudaError_t e__ = (call);                                                                             \
        if (e__ != cudaSuccess) return fail(ln_fail(ctx, LN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__))); \
    } while (0)
    LN_Y(cudaMemsetAsync(hist, 0, sz_hist, ctx->stream));
    if (p.cache_stride != (unsigned)p.total_ca * (unsigned)p.classes) LN_Y(cudaMemsetAsync(cache, 0, sz_cache, ctx->stream));  // zero the per-image padding
    LN_Y(cudaMemsetAsync(band_fill, 0, sz_fill, ctx->stream));
    LN_Y(cudaMemsetAsync(flags, 0, 256, ctx->stream));
    LN_Y(cudaMemcpyAsync(dims, image_w, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    LN_Y(cudaMemcpyAsync(dims + B, image_h, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    yolo_init_states_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(states, dims, dims + B, B);
    ctx->launches++;

    const size_t nms_smem = (size_t)p.band_max * 8 + (size_t)(p.k_eff + kChunk) * sizeof(float4) + (size_t)kChunk * (kChunk / 32) * 4 +
                            (size_t)(p.k_eff + kChunk) * 4 + (size_t)kChunk * 8 + 64;
    LN_Y(cudaFuncSetAttribute(yolo_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)nms_smem));
    const dim3 scan_grid((p.total_ca + 255) / 256, B);
    const dim3 flat_grid((unsigned)(((int64_t)p.total_ca * p.classes + kFlatChunk - 1) / kFlatChunk), B);
    int* h_flags = ctx->h_status + 4;
    const int max_rounds = 4096;
    int round = 0;
    const bool dbg = getenv("LN_DEBUG_NMS") != nullptr;
    auto now = []() { timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts); return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6; };
    double t_sel = 0, t_nms = 0;
    int n_levels = 0;
    for (; round < max_rounds; ++round) {
        const double ta = dbg ? now() : 0;
        for (int level = 0; level < kLevels; ++level) {
            ++n_levels;
            if (round == 0 && level == 0) yolo_scan_kernel<0, true><<<scan_grid, 256, 0, ctx->stream>>>(p, states, hist, band, band_fill, cache);
            else yolo_scan_cached_kernel<0><<<flat_grid, 256, 0, ctx->stream>>>(p, states, hist, band, band_fill, cache);
            yolo_select_kernel<<<B, 256, 0, ctx->stream>>>(p, states, hist, flags);
            ctx->launches += 2;
            LN_Y(cudaMemcpyAsync(h_flags, flags, 4, cudaMemcpyDeviceToHost, ctx->stream));
            LN_Y(cudaMemsetAsync(flags, 0, 4, ctx->stream));
            LN_Y(cudaStreamSynchronize(ctx->stream));
            if (h_flags[0] == 0) break;
        }
        const double tb = dbg ? now() : 0;
        t_sel += tb - ta;
        yolo_scan_cached_kernel<1><<<flat_grid, 256, 0, ctx->stream>>>(p, states, hist, band, band_fill, cache);
        if (dbg) { cudaStreamSynchronize(ctx->stream); const double tc = now(); fprintf(stderr, "[ln_yolo] collect %.3f ms\n", tc - tb); }
        const double td = dbg ? now() : 0;
        yolo_nms_kernel<<<B, 1024, nms_smem, ctx->stream>>>(p, states, band, band_fill, kept_box, kept_cls, records, flags + 1);
        ctx->launches += 2;
        LN_Y(cudaMemcpyAsync(h_flags, flags + 1, 4, cudaMemcpyDeviceToHost, ctx->stream));
        LN_Y(cudaMemsetAsync(flags + 1, 0, 4, ctx->stream));
        LN_Y(cudaStreamSynchronize(ctx->stream));
        if (dbg) t_nms += now() - td;
        if (h_flags[0] == 0) break;
    }
    if (dbg) fprintf(stderr, "[ln_yolo] batch %d: %d rounds, %d selection passes (%.3f ms), nms kernels %.3f ms, band_max %d, k_eff %d\n", B, round + 1, n_levels, t_sel, t_nms, p.band_max, p.k_eff);
    if (round == max_rounds) return fail(ln_fail(ctx, LN_ERR_TIMEOUT, "ln_yolo_decode_nms: NMS did not finish in %d rounds", max_rounds));
    yolo_counts_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(states, counts, B, p.max_per_image);
    ctx->launches++;
    LN_Y(cudaGetLastError());
    LN_Y(cudaMemcpyAsync(counts_host, counts, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LN_Y(cudaMemcpyAsync(records_host, records, (size_t)B * p.max_per_image * sizeof(ln_detection), cudaMemcpyDeviceToHost, ctx->stream));
    LN_Y(cudaStreamSynchronize(ctx->stream));
#undef LN_Y
    ln_pool_free(ctx, scratch, total);
    return LN_OK;
}

// ---- decode + NMS without any allocation ------------------------------------------------------------
// Working memory of ln_yolo_decode_nms_noalloc: a fixed array that is part of the loaded module.  Every GPU
// that loads this library carries these 64 MiB until the process exits, whether or not the entry point is used.
#define LN_NOALLOC_SCRATCH_BYTES (64u * 1024u * 1024u)
static __device__ __align__(256) unsigned char ln_noalloc_scratch[LN_NOALLOC_SCRATCH_BYTES];
// Device address of the array above, per device ordinal.  In host code the name `ln_noalloc_scratch` is only a
// stand-in for the symbol, not a pointer a kernel could use; the address has to be asked for, once per device.
static unsigned char* g_noalloc_ptr[64] = {nullptr};

int32_t ln_yolo_decode_nms_noalloc(ln_ctx* ctx, const ln_yolo_head* heads, int32_t n_heads, int32_t net_w, int32_t net_h, const int32_t* image_w,
                                   const int32_t* image_h, const ln_detect_options* opts, ln_detection* records_host, int32_t* counts_host) {
    const char* who = "ln_yolo_decode_nms_noalloc";
    if (!ctx || !heads || !image_w || !image_h || !opts || !records_host || !counts_host) return ln_fail(ctx, LN_ERR_ARG, "%s: NULL argument", who);
    if (opts->max_per_image < 1) return ln_fail(ctx, LN_ERR_ARG, "%s: max_per_image must be positive", who);
    if (ctx->device < 0 || ctx->device >= 64) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "%s: device ordinal %d is outside the table of 64", who, ctx->device);
    YoloParams p;
    int rc = fill_params(ctx, &p, heads, n_heads, net_w, net_h, who);
    if (rc) return rc;
    p.thr = opts->confidence_threshold;
    p.nms_thr = opts->nms_threshold;
    p.letterbox = opts->letterbox;
    p.max_per_image = opts->max_per_image;
    p.k_eff = opts->top_k > 0 && opts->top_k < opts->max_per_image ? opts->top_k : opts->max_per_image;
    p.band_max = kBandMaxSmall;
    if (p.k_eff > 4096) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "%s: at most 4096 detections per image (top_k / max_per_image)", who);
    for (int i = 0; i < p.batch; ++i)
        if (image_w[i] <= 0 || image_h[i] <= 0) return ln_fail(ctx, LN_ERR_ARG, "image dimensions must be positive for network detection decoding");
    const int B = p.batch;
    const size_t sz_states = (size_t)ln_round_up((int64_t)B * sizeof(ImgState), 256);
    const size_t sz_hist = (size_t)B * kBins * 4;
    const size_t sz_band = (size_t)B * p.band_max * 8;
    const size_t sz_fill = (size_t)ln_round_up((int64_t)B * 4, 256);
    const size_t sz_kbox = (size_t)B * p.k_eff * sizeof(float4);
    const size_t sz_kcls = (size_t)ln_round_up((int64_t)B * p.k_eff * 4, 256);
    const size_t sz_rec = (size_t)ln_round_up((int64_t)B * p.max_per_image * sizeof(ln_detection), 256);
    const size_t sz_dims = (size_t)ln_round_up((int64_t)B * 8, 256);
    const size_t sz_cnt = (size_t)ln_round_up((int64_t)B * 4, 256);
    p.cache_stride = (unsigned)ln_round_up((int64_t)p.total_ca * p.classes, 4);
    const size_t sz_cache = (size_t)ln_round_up((int64_t)B * p.cache_stride * 4, 256);
    const size_t total = sz_states + sz_hist + sz_band + sz_fill + sz_kbox + sz_kcls + sz_rec + sz_dims + sz_cnt + sz_cache + 256;
    if (total > (size_t)LN_NOALLOC_SCRATCH_BYTES)
        return ln_fail(ctx, LN_ERR_UNSUPPORTED,
                       "%s: this call needs %zu bytes of working memory (batch %d, %d candidates per image, %d records per image) but the fixed "
                       "array holds %u; use a smaller batch, fewer records, or ln_yolo_decode_nms",
                       who, total, B, p.total_ca * p.classes, p.max_per_image, LN_NOALLOC_SCRATCH_BYTES);
    cudaSetDevice(ctx->device);
    if (!g_noalloc_ptr[ctx->device]) {
        // once per device, with that device current: the address of the module's array on this device
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, ln_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return ln_fail(ctx, LN_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", who, cudaGetErrorString(e));
        g_noalloc_ptr[ctx->device] = (unsigned char*)ptr;
    }
    unsigned char* q = g_noalloc_ptr[ctx->device];
    ImgState* states = (ImgState*)q; q += sz_states;
    unsigned* hist = (unsigned*)q; q += sz_hist;
    unsigned long long* band = (unsigned long long*)q; q += sz_band;
    int* band_fill = (int*)q; q += sz_fill;
    float4* kept_box = (float4*)q; q += sz_kbox;
    int* kept_cls = (int*)q; q += sz_kcls;
    ln_detection* records = (ln_detection*)q; q += sz_rec;
    int* dims = (int*)q; q += sz_dims;
    int* counts = (int*)q; q += sz_cnt;
    unsigned* cache = (unsigned*)q; q += sz_cache;
    int* flags = (int*)q;
#define LN_Z(call)                                                                                     \
    do {                                                                                               \
        cudaError_t e__ = (call);                                                                      \
        if (e__ != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
    } while (0)
    // the array keeps whatever the previous call left: clear everything the kernels expect to start at zero
    LN_Z(cudaMemsetAsync(hist, 0, sz_hist, ctx->stream));
    LN_Z(cudaMemsetAsync(band_fill, 0, sz_fill, ctx->stream));
    LN_Z(cudaMemsetAsync(flags, 0, 256, ctx->stream));
    if (p.cache_stride != (unsigned)p.total_ca * (unsigned)p.classes) LN_Z(cudaMemsetAsync(cache, 0, sz_cache, ctx->stream));
    LN_Z(cudaMemcpyAsync(dims, image_w, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    LN_Z(cudaMemcpyAsync(dims + B, image_h, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    yolo_init_states_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(states, dims, dims + B, B);
    ctx->launches++;
    const size_t nms_smem = (size_t)p.band_max * 8 + (size_t)(p.k_eff + kChunk) * sizeof(float4) + (size_t)kChunk * (kChunk / 32) * 4 +
                            (size_t)(p.k_eff + kChunk) * 4 + (size_t)kChunk * 8 + 64;
    LN_Z(cudaFuncSetAttribute(yolo_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)nms_smem));
    const dim3 scan_grid((p.total_ca + 255) / 256, B);
    const dim3 flat_grid((unsigned)(((int64_t)p.total_ca * p.classes + kFlatChunk - 1) / kFlatChunk), B);
    int* h_flags = ctx->h_status + 4;
    const int max_rounds = 4096;
    int round = 0;
    for (; round < max_rounds; ++round) {
        for (int level = 0; level < kLevels; ++level) {
            if (round == 0 && level == 0) yolo_scan_kernel<0, true><<<scan_grid, 256, 0, ctx->stream>>>(p, states, hist, band, band_fill, cache);
            else yolo_scan_cached_kernel<0><<<flat_grid, 256, 0, ctx->stream>>>(p, states, hist, band, band_fill, cache);
            yolo_select_kernel<<<B, 256, 0, ctx->stream>>>(p, states, hist, flags);
            ctx->launches += 2;
            LN_Z(cudaMemcpyAsync(h_flags, flags, 4, cudaMemcpyDeviceToHost, ctx->stream));
            LN_Z(cudaMemsetAsync(flags, 0, 4, ctx->stream));
            LN_Z(cudaStreamSynchronize(ctx->stream));
            if (h_flags[0] == 0) break;
        }
        yolo_scan_cached_kernel<1><<<flat_grid, 256, 0, ctx->stream>>>(p, states, hist, band, band_fill, cache);
        yolo_nms_kernel<<<B, 1024, nms_smem, ctx->stream>>>(p, states, band, band_fill, kept_box, kept_cls, records, flags + 1);
        ctx->launches += 2;
        LN_Z(cudaMemcpyAsync(h_flags, flags + 1, 4, cudaMemcpyDeviceToHost, ctx->stream));
        LN_Z(cudaMemsetAsync(flags + 1, 0, 4, ctx->stream));
        LN_Z(cudaStreamSynchronize(ctx->stream));
        if (h_flags[0] == 0) break;
    }
    if (round == max_rounds) return ln_fail(ctx, LN_ERR_TIMEOUT, "%s: NMS did not finish in %d rounds", who, max_rounds);
    yolo_counts_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(states, counts, B, p.max_per_image);
    ctx->launches++;
    LN_Z(cudaGetLastError());
    LN_Z(cudaMemcpyAsync(counts_host, counts, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LN_Z(cudaMemcpyAsync(records_host, records, (size_t)B * p.max_per_image * sizeof(ln_detection), cudaMemcpyDeviceToHost, ctx->stream));
    LN_Z(cudaStreamSynchronize(ctx->stream));
#undef LN_Z
    return LN_OK;
}

int32_t ln_yolo_decode_only(ln_ctx* ctx, const ln_yolo_head* heads, int32_t n_heads, int32_t image_index, int32_t net_w, int32_t net_h,
                            int32_t image_w, int32_t image_h, float confidence_threshold, int32_t letterbox, ln_detection* records_host,
                            int64_t capacity, int64_t* count) {
    if (!ctx || !heads || !records_host || !count) return ln_fail(ctx, LN_ERR_ARG, "ln_yolo_decode_only: NULL argument");
    YoloParams p;
    int rc = fill_params(ctx, &p, heads, n_heads, net_w, net_h, "ln_yolo_decode_only");
    if (rc) return rc;
    if (image_index < 0 || image_index >= p.batch) return ln_fail(ctx, LN_ERR_ARG, "batch index %d is outside YOLO head batch %d", image_index, p.batch);
    if (image_w <= 0 || image_h <= 0) return ln_fail(ctx, LN_ERR_ARG, "image dimensions must be positive for network detection decoding");
    p.thr = confidence_threshold;
    p.letterbox = letterbox;
    cudaSetDevice(ctx->device);
    const int n = p.total_ca;
    int* d_counts = (int*)ln_pool_alloc(ctx, (size_t)n * 4);
    long long* d_off = (long long*)ln_pool_alloc(ctx, (size_t)n * 8);
    ln_detection* d_out = (ln_detection*)ln_pool_alloc(ctx, (size_t)(capacity > 0 ? capacity : 1) * sizeof(ln_detection));
    auto cleanup = [&]() {
        ln_pool_free(ctx, d_counts, (size_t)n * 4);
        ln_pool_free(ctx, d_off, (size_t)n * 8);
        ln_pool_free(ctx, d_out, (size_t)(capacity > 0 ? capacity : 1) * sizeof(ln_detection));
    };
    if (!d_counts || !d_off || !d_out) { cleanup(); return LN_ERR_CUDA; }
    yolo_decode_count_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(p, image_index, d_counts);
    ctx->launches++;
    std::vector<int> h_counts((size_t)n);
    std::vector<long long> h_off((size_t)n);
    cudaError_t e = cudaMemcpyAsync(h_counts.data(), d_counts, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    long long total = 0;
    for (int i = 0; i < n; ++i) { h_off[i] = total; total += h_counts[i]; }
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_off, h_off.data(), (size_t)n * 8, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        yolo_decode_write_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(p, image_index, image_w, image_h, d_off, d_out, capacity);
        ctx->launches++;
        e = cudaGetLastError();
    }
    const long long ncopy = total < capacity ? total : capacity;
    if (e == cudaSuccess && ncopy > 0) e = cudaMemcpyAsync(records_host, d_out, (size_t)ncopy * sizeof(ln_detection), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cleanup();
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "ln_yolo_decode_only: %s", cudaGetErrorString(e));
    *count = total;
    return LN_OK;
}

}  // extern "C"
