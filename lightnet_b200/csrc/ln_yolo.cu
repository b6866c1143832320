// [yolo] decode + per-class greedy NMS on the device.
//
// Reference semantics (lightnet-train/src/detect.rs): decode_yolo_head (:934-1016) emits one candidate per
// (head, anchor, cell, class) with objectness > thr and confidence = objectness * class_prob > thr, in that
// order; the list is stably sorted by confidence descending (:107) and apply_nms (:1449-1484) walks it: a
// candidate survives unless an earlier survivor of the same class overlaps it with IoU > nms_thr.
//
// Device formulation.  Every candidate gets the 64-bit key (order-preserving confidence bits << 32) |
// ~emission_index; descending key order is exactly the reference's sorted order, ties included.  Greedy NMS
// only ever needs candidates in that order, and only until top_k survivors exist, so they are consumed from
// the top in two stages:
//
//   pool  - two passes over the head tensors.  The first histograms the top 12 key bits of every candidate;
//           a walk down the histogram fixes a key `pool_lo` such that the candidates at or above it are a few
//           times what the survivors still wanted can need; the second pass writes exactly those keys to a
//           compact per-image pool (or, when they fit, straight into the band).  Should one histogram bin hold
//           more than a pool can (massive ties), the selection descends a digit with another pass.
//   band  - inside the pool a radix selection over the compact keys (cheap: the pool sits in L2) cuts bands
//           that fit in shared memory; each band is sorted (bitonic) and resolved by one CTA per image: every
//           512-candidate chunk is tested against the survivors so far, a 512 x 512 same-class IoU bitmask is
//           built, and one warp resolves it with shuffles.
//
// An image stops as soon as it has top_k survivors or runs out of candidates; a pool that is used up before
// that is followed by the next one further down.  The head tensors are the only large input: they are read
// twice per pool, and nothing of their size is written.
//
// Most of the candidates only need their histogram bin, not their exact bits.  The passes over the heads
// therefore evaluate the class sigmoid with the hardware ex2 / rcp approximations first and fall back to the
// exact evaluation only when the approximate key is within kKeySlack units of a boundary that matters (a bin
// edge, the threshold, the ends of the range being collected).  Everything that is written anywhere -- pool
// and band keys, records -- comes from the exact evaluation: sigmoid, box decode and IoU use single IEEE-754
// operations in the reference's evaluation order, so a CPU evaluating the same expressions gets the same bits.
#include <cooperative_groups.h>

#include <cstdlib>
#include <ctime>

#include "ln_conv_plan.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kMaxHeads = 8;
constexpr int kBandMaxLarge = 16384;  // candidates of one band (sorted in shared memory) when at most 1024 survivors are wanted
constexpr int kBandMaxSmall = 8192;   // ... when more are wanted (their boxes need the room)
constexpr int kChunk = 512;      // candidates resolved per bitmask step
constexpr int kBins = 4096;      // 12-bit radix digits
constexpr unsigned kPoolChunk = 8192;  // pool keys one block of the pool passes walks
constexpr int kLevels = 6;       // 5 x 12 bits + 4 bits = 64
// Largest distance, in units of the 32-bit confidence key, assumed between the key of the approximate score and
// the key of the exact one.  The approximations are good to a few units (measured by ln_debug_score_key_error).
constexpr unsigned kKeySlack = 256;
constexpr long long kPoolBytesTarget = 1ll << 30;  // pools of one call together, unless every candidate fits in less

enum { PHASE_POOL = 0, PHASE_FILL = 1, PHASE_SELECT = 2, PHASE_BAND = 3, PHASE_DONE = 4 };
enum { FLAG_SELECT_PENDING = 0, FLAG_ACTIVE = 1, FLAG_POOL_PENDING = 2, FLAG_NEED_POOL = 3 };

struct HeadDev {
    const float* raw;  // [batch][n_anchor*(5+classes)][gh*gw]
    int gw, gh, classes, n_anchor, new_coords;
    // 0 = [yolo]; 1 = activated [yolox] head; 2 = predecoded distribution head ([ppyoloe] / [yolonas]).  Kinds 1 and 2 hold
    // probabilities already (new_coords = 1: values are used as they are) and have one box per cell.
    int kind;
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
    int pool_max;       // capacity of one pool
    int hist_stride;    // the first histogram of a pool looks at every hist_stride-th block of 256 (anchor, cell) slots
};

struct ImgState {
    unsigned long long hi;       // keys >= hi have been consumed
    unsigned long long lo;       // current band is [lo, hi)
    unsigned long long prefix;   // digits fixed so far by the radix selection in progress (pool or band)
    unsigned long long pool_lo;  // the pool holds every candidate in [pool_lo, hi at the time it was filled)
    int level, phase, cap, above, band_count, kept, exhausted, img_w, img_h;
    int last_gain;   // survivors the previous band added
    int direct;      // the pool being filled is small enough to be the band itself
    int pool_count;  // keys in the pool
    int sampled;     // the histogram in progress is an estimate from a sample of the slots
    // band selection inside a pool starts at the first digit on which the pool's keys differ (all earlier digits = start_prefix)
    int start_level, fresh;
    unsigned long long start_prefix;
};

__device__ __forceinline__ int level_shift(int l) { return l < 5 ? 52 - 12 * l : 0; }
__device__ __forceinline__ int level_bits(int l) { return l < 5 ? 12 : 4; }

__device__ __forceinline__ float head_act(float raw, int new_coords) { return new_coords ? raw : ln_det_sigmoid(raw); }
// The objectness factor of a score.  The distribution heads gate on max(class, objectness * class) (detect.rs:1158-1162), which
// is the class score itself for an objectness in [0, 1]: their factor is 1 (a product with 1 is exact).
__device__ __forceinline__ float score_obj(const HeadDev& h, float raw_obj) { return h.kind == 2 ? 1.0f : head_act(raw_obj, h.new_coords); }

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
    float bx, by, bw, bh;
    const float aw = h.anchors[2 * a], ah = h.anchors[2 * a + 1];
    if (h.kind == 2) {  // final centre-size box of modern_yolo_predecode (dense_loss.rs:788)
        bx = tx; by = ty; bw = tw; bh = th;
    } else if (h.kind == 1) {  // decode_yolox_box (lightnet-layers/src/modern_yolo/cpu.rs:461-475), sanitised like cpu.rs:212-217
        const float cw = fminf(fmaxf(ln_finite_or_zero(tw), -10.0f), 10.0f), ch = fminf(fmaxf(ln_finite_or_zero(th), -10.0f), 10.0f);
        bx = ln_finite_or_zero(__fdiv_rn(__fadd_rn((float)col, ln_finite_or_zero(tx)), (float)h.gw));
        by = ln_finite_or_zero(__fdiv_rn(__fadd_rn((float)row, ln_finite_or_zero(ty)), (float)h.gh));
        bw = fmaxf(ln_finite_or_zero(__fdiv_rn(ln_det_expf(cw), (float)h.gw)), 1e-6f);
        bh = fmaxf(ln_finite_or_zero(__fdiv_rn(ln_det_expf(ch), (float)h.gh)), 1e-6f);
    } else {
    bx = __fdiv_rn(__fsub_rn(__fadd_rn((float)col, __fmul_rn(s, head_act(tx, h.new_coords))), half), (float)h.gw);
    by = __fdiv_rn(__fsub_rn(__fadd_rn((float)row, __fmul_rn(s, head_act(ty, h.new_coords))), half), (float)h.gh);
    if (h.new_coords) {
        bw = __fdiv_rn(__fmul_rn(__fmul_rn(__fmul_rn(tw, tw), 4.0f), aw), nw);
        bh = __fdiv_rn(__fmul_rn(__fmul_rn(__fmul_rn(th, th), 4.0f), ah), nh);
    } else {
        bw = __fdiv_rn(__fmul_rn(ln_det_expf(tw), aw), nw);
        bh = __fdiv_rn(__fmul_rn(ln_det_expf(th), ah), nh);
    }
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

// Band size wanted next: four candidates per survivor still wanted, or more when the previous band showed heavier suppression.
__device__ __forceinline__ int band_cap(const YoloParams& p, const ImgState& st) {
    long long want = 4ll * (p.k_eff - st.kept);
    if (st.last_gain >= 0) {
        const long long per = ((long long)st.band_count * 3 / 2) / (st.last_gain > 0 ? st.last_gain : 1) + 1;
        if (per > 4) want = per * (p.k_eff - st.kept);
    }
    return want < 1024 ? 1024 : (want > p.band_max ? p.band_max : (int)want);
}

// Confidence key of objectness * sigmoid(x) as an interval [klo, khi] that contains the exact key (valid for thresholds
// >= 1e-30, see approx_ok below).  Branch-free on the common path:
//   x >= 17   the exact sigmoid is 1, the score is the objectness itself: klo == khi
//   x <= -80  ex2 overflows, the approximate score is 0; the exact one is below 2e-35: both far under the threshold
//   NaN       not handled here: callers send NaN logits to the exact path
__device__ __forceinline__ void approx_score_key(float obj, float x, unsigned& klo, unsigned& khi) {
    const bool sat = x >= 17.0f;
    const float s = sat ? obj : obj * ln_rcp_ftz(1.0f + ln_ex2_ftz(x * -1.44269504f));
    const unsigned k = __float_as_uint(s) | 0x80000000u;  // s >= +0 (or NaN)
    const unsigned d = sat ? 0u : kKeySlack;
    klo = k - d;
    khi = k + d;
}

// The same interval for either kind of head: heads with new_coords take the class value as it is, so their score is one
// exact product and the interval a single key (NaN scores are left to the exact evaluation, which drops them).
__device__ __forceinline__ bool score_key_interval(float obj, float x, int new_coords, bool approx_ok, unsigned& klo, unsigned& khi) {
    if (new_coords) {
        const float conf = __fmul_rn(obj, x);
        klo = khi = conf_key(conf);
        return approx_ok && conf == conf;
    }
    approx_score_key(obj, x, klo, khi);
    return approx_ok && x == x;  // a NaN logit goes to the exact evaluation, whose clamps decide what it means
}

constexpr int kWarpBuf = 512;  // keys one warp of the fill pass buffers in shared memory before it reserves space in the pool

// Range of keys one pass over the heads is interested in, [rlo, rhi] inclusive, from the state of the image.
struct ScanRange {
    unsigned long long rlo, rhi;
    unsigned rlo_ck, rhi_ck;
};
template <int MODE>
__device__ __forceinline__ ScanRange scan_range(const ImgState& st) {
    ScanRange r;
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    r.rhi = st.hi - 1ull;  // hi >= 1 whenever an image is still active
    if (MODE == 1) r.rlo = st.pool_lo;
    else if (st.level == 0) r.rlo = 0ull;
    else {
        r.rlo = st.prefix << (shift + bits);
        const unsigned long long pend = r.rlo | ((1ull << (shift + bits)) - 1ull);
        if (pend < r.rhi) r.rhi = pend;
    }
    r.rlo_ck = (unsigned)(r.rlo >> 32);
    r.rhi_ck = (unsigned)(r.rhi >> 32);
    return r;
}

// Exact key of one candidate, or 0 when it is not a candidate inside [rlo, rhi].
__device__ __forceinline__ unsigned long long exact_key_in_range(const YoloParams& p, const ScanRange& r, float obj, float x, int new_coords,
                                                                 unsigned ca, unsigned c) {
    const float conf = __fmul_rn(obj, head_act(x, new_coords));
    if (!(conf > p.thr)) return 0ull;
    const unsigned eidx = ca * (unsigned)p.classes + c;
    const unsigned long long key = ((unsigned long long)conf_key(conf) << 32) | (unsigned long long)(0xFFFFFFFFu - eidx);
    return (key < r.rlo || key > r.rhi) ? 0ull : key;  // a real key is never 0: its confidence bits are at least 0x80000000
}

// First pass over the head tensors for the images that need a pool: histogram of digit `level` (under `prefix`) of the
// unconsumed candidates (keys < hi).  One thread per (anchor, cell), all classes; blockIdx.y = image.  The common path of
// the class loop is branch-free: the flags of a score are computed unconditionally and only the rare score that needs the
// exact evaluation leaves it.
__global__ void __launch_bounds__(256) yolo_head_hist_kernel(const __grid_constant__ YoloParams p, const ImgState* __restrict__ states,
                                                             unsigned* __restrict__ hist) {
    const int img = blockIdx.y;
    const ImgState st = states[img];
    if (st.phase != PHASE_POOL) return;
    // an estimate is enough to place the pool's lower bound (the fill pass is exact whatever the bound): sampled images
    // histogram one block in hist_stride, offset by the image index
    if (st.sampled && (int)(blockIdx.x % p.hist_stride) != img % p.hist_stride) return;
    __shared__ unsigned s_hist[kBins + 1];  // slot kBins swallows the first, empty run of every thread
    for (int i = threadIdx.x; i <= kBins; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    const ScanRange r = scan_range<0>(st);
    const unsigned kthr = conf_key(p.thr);
    const bool approx_ok = p.thr >= 1e-30f;  // below that the exact exponential's clamp decides candidates
    const bool level0 = st.level == 0;
    const int ca = blockIdx.x * blockDim.x + threadIdx.x;
    if (ca < p.total_ca) {
        const HeadDev& h = p.heads[find_head(p, ca)];
        const int stride = h.gw * h.gh, new_coords = h.new_coords;
        const int epa = h.classes + 5, local = ca - h.ca_base;
        const int a = local / stride, idx = local - a * stride;
        const float* img_raw = h.raw + (size_t)img * h.n_anchor * epa * stride;
        const float obj = score_obj(h, __ldg(img_raw + (size_t)(a * epa + 4) * stride + idx));
        const float* __restrict__ cls_raw = img_raw + (size_t)(a * epa + 5) * stride + idx;
        if (obj > p.thr) {
            // consecutive classes often fall into the same bin (always, when scores saturate): runs are counted in registers
            unsigned run_bin = kBins, run_len = 0;
            // eight class logits are loaded before any of them is used: eight independent loads in flight per thread
            for (int c0 = 0; c0 < p.classes; c0 += 8) {
                float xs[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) xs[j] = c0 + j < p.classes ? __ldg(cls_raw + (size_t)j * stride) : 0.0f;
                cls_raw += (size_t)8 * stride;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float x = xs[j];
                    unsigned klo, khi;
                    const bool usable = score_key_interval(obj, x, new_coords, approx_ok, klo, khi);
                    const bool out = khi <= kthr || klo > r.rhi_ck || khi < r.rlo_ck;  // certainly not a candidate of interest
                    unsigned bin = klo >> 20;
                    const bool certain = level0 && klo > kthr && khi < r.rhi_ck && bin == (khi >> 20);  // the bin is all this pass needs
                    bool count = usable && !out && certain;
                    if (c0 + j < p.classes && !(usable && (out || certain))) {  // rare
                        const unsigned long long key = exact_key_in_range(p, r, obj, x, new_coords, (unsigned)ca, (unsigned)(c0 + j));
                        count = key != 0ull;
                        bin = (unsigned)(key >> shift) & ((1u << bits) - 1u);
                    }
                    count = count && c0 + j < p.classes;
                    const bool same = bin == run_bin;
                    if (count && !same) {
                        atomicAdd(&s_hist[run_bin], run_len);
                        run_bin = bin;
                        run_len = 0;
                    }
                    run_len += count ? 1u : 0u;
                }
            }
            atomicAdd(&s_hist[run_bin], run_len);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBins; i += blockDim.x)
        if (s_hist[i]) atomicAdd(&hist[(size_t)img * kBins + i], s_hist[i]);
}

// Second pass over the heads: write the exact keys of the candidates in [pool_lo, hi) to the pool, or to the band when
// `direct`.  A block first lists the (anchor, cell) slots of its 256 whose objectness reaches the range at all (a class
// probability never exceeds 1 where a sigmoid makes it), then walks (class, listed slot) pairs with all its threads, so
// that a few qualifying cells do not leave most lanes idle.  Keys are buffered per warp in shared memory and written
// out with one reservation per few hundred keys.
__global__ void __launch_bounds__(256) yolo_head_fill_kernel(const __grid_constant__ YoloParams p, const ImgState* __restrict__ states,
                                                             unsigned long long* __restrict__ band, int* __restrict__ band_fill,
                                                             unsigned long long* __restrict__ pool, int* __restrict__ pool_fill,
                                                             unsigned long long* __restrict__ key_and_or) {
    const int img = blockIdx.y;
    const ImgState st = states[img];
    if (st.phase != PHASE_FILL) return;
    __shared__ unsigned long long s_buf[8 * kWarpBuf];
    __shared__ int s_cnt[8];
    __shared__ const float* s_ptr[256];
    __shared__ float s_obj[256];
    __shared__ int s_stride[256];
    __shared__ int s_ca[256];   // slot index, with the head's new_coords flag in bit 31
    __shared__ int s_n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) s_cnt[warp] = 0;
    if (threadIdx.x == 0) s_n = 0;
    __syncthreads();
    const ScanRange r = scan_range<1>(st);
    const unsigned kthr = conf_key(p.thr);
    const bool approx_ok = p.thr >= 1e-30f;
    unsigned long long* dst = st.direct ? band + (size_t)img * p.band_max : pool + (size_t)img * p.pool_max;
    int* fill = st.direct ? band_fill + img : pool_fill + img;
    const int dst_cap = st.direct ? p.band_max : p.pool_max;
    const int ca = blockIdx.x * blockDim.x + threadIdx.x;
    if (ca < p.total_ca) {
        const HeadDev& h = p.heads[find_head(p, ca)];
        const int stride = h.gw * h.gh, new_coords = h.new_coords;
        const int epa = h.classes + 5, local = ca - h.ca_base;
        const int a = local / stride, idx = local - a * stride;
        const float* img_raw = h.raw + (size_t)img * h.n_anchor * epa * stride;
        const float obj = score_obj(h, __ldg(img_raw + (size_t)(a * epa + 4) * stride + idx));
        if (obj > p.thr && (new_coords || conf_key(obj) >= r.rlo_ck)) {
            const int slot = atomicAdd(&s_n, 1);
            s_ptr[slot] = img_raw + (size_t)(a * epa + 5) * stride + idx;
            s_obj[slot] = obj;
            s_stride[slot] = stride;
            s_ca[slot] = ca | (new_coords ? (int)0x80000000 : 0);
        }
    }
    __syncthreads();
    const int n_listed = s_n;
    if (n_listed == 0) return;
    unsigned long long t_and = ~0ull, t_or = 0ull;  // over the keys this thread emits
    auto emit = [&](unsigned long long key) {
        const int slot = atomicAdd(&s_cnt[warp], 1);  // stays below kWarpBuf, see the flush conditions
        s_buf[warp * kWarpBuf + slot] = key;
        t_and &= key;
        t_or |= key;
    };
    auto publish_and_or = [&]() {
        for (int o = 16; o > 0; o >>= 1) {
            t_and &= __shfl_xor_sync(0xffffffffu, t_and, o);
            t_or |= __shfl_xor_sync(0xffffffffu, t_or, o);
        }
        if (lane == 0 && t_or != 0ull) { atomicAnd(&key_and_or[2 * img], t_and); atomicOr(&key_and_or[2 * img + 1], t_or); }
    };
    auto flush_if = [&](int limit, bool last) {
        // the warp writes its buffered keys out when the next step could overflow the buffer, and at the end
        __syncwarp();
        const int n = s_cnt[warp];
        if (n > limit || (n > 0 && last)) {
            int at = 0;
            if (lane == 0) at = atomicAdd(fill, n);
            at = __shfl_sync(0xffffffffu, at, 0);
            for (int k = lane; k < n; k += 32)
                if (at + k < dst_cap) dst[at + k] = s_buf[warp * kWarpBuf + k];
            __syncwarp();
            if (lane == 0) s_cnt[warp] = 0;
        }
        __syncwarp();
    };
    if (n_listed >= 64) {
        // many listed slots: thread t takes listed slot t and walks its classes, eight loads in flight
        if (warp * 32 >= n_listed) return;
        const bool have = (int)threadIdx.x < n_listed;
        const int j = have ? (int)threadIdx.x : 0;
        const float obj = s_obj[j];
        const int new_coords = s_ca[j] < 0 ? 1 : 0, stride = s_stride[j];
        const unsigned cell = (unsigned)s_ca[j] & 0x7FFFFFFFu;
        const float* __restrict__ cls_raw = s_ptr[j];
        for (int c0 = 0; c0 < p.classes; c0 += 8) {
            if (have) {
                float xs[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) xs[q] = c0 + q < p.classes ? __ldg(cls_raw + (size_t)q * stride) : 0.0f;
                cls_raw += (size_t)8 * stride;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float x = xs[q];
                    unsigned klo, khi;
                    const bool out = score_key_interval(obj, x, new_coords, approx_ok, klo, khi) && (khi <= kthr || khi < r.rlo_ck || klo > r.rhi_ck);
                    if (!out && c0 + q < p.classes) {
                        const unsigned long long key = exact_key_in_range(p, r, obj, x, new_coords, cell, (unsigned)(c0 + q));
                        if (key != 0ull) emit(key);
                    }
                }
            }
            flush_if(kWarpBuf - 256, c0 + 8 >= p.classes);  // a step adds at most 8 x 32 keys
        }
        publish_and_or();
        return;
    }
    // few listed slots: all threads share the (class, listed slot) pairs
    const int items = n_listed * p.classes;
    for (int base = 0; base < items; base += 256) {  // uniform trip count
        const int i = base + (int)threadIdx.x;
        if (i < items) {
            const int c = i / n_listed, j = i - c * n_listed;
            const float obj = s_obj[j];
            const int new_coords = s_ca[j] < 0 ? 1 : 0;
            const unsigned cell = (unsigned)s_ca[j] & 0x7FFFFFFFu;
            const float x = __ldg(s_ptr[j] + (size_t)c * s_stride[j]);
            bool maybe = true;
            unsigned klo, khi;
            if (score_key_interval(obj, x, new_coords, approx_ok, klo, khi)) maybe = !(khi <= kthr || khi < r.rlo_ck || klo > r.rhi_ck);
            if (maybe) {
                const unsigned long long key = exact_key_in_range(p, r, obj, x, new_coords, cell, (unsigned)c);
                if (key != 0ull) emit(key);
            }
        }
        flush_if(kWarpBuf - 32, base + 256 >= items);  // a step adds at most 32 keys
    }
    publish_and_or();
}

// Loads the histogram of one image top bin first into shared memory (and zeroes it in global memory);
// s_part[t] = sum of the 16 slots thread t loaded.  Slot 0 is the top bin.
__device__ __forceinline__ void load_hist_desc(unsigned* h, int nb, unsigned* s_h, unsigned* s_part) {
    const int per = kBins / 256;
    unsigned sum = 0;
    for (int j = 0; j < per; ++j) {
        const int slot = threadIdx.x * per + j;
        const int bin = nb - 1 - slot;
        const unsigned v = bin >= 0 ? h[bin] : 0u;
        s_h[slot] = v;
        sum += v;
        if (bin >= 0) h[bin] = 0u;
    }
    s_part[threadIdx.x] = sum;
    __syncthreads();
}

// One block per image that needs a pool: walk the digit histogram from the top until the candidates counted reach the
// band size wanted; everything from that bin up is the pool.  A bin too large for a pool is descended into.
// With a sampled histogram the counts are estimates (scaled by the sampling stride): the target is doubled, sizes are
// compared with a margin of one half, and an image whose boundary bin looks too large for a pool starts over with the
// full histogram.  The fill pass counts exactly; should it overflow all the same, the image starts over as well.
__global__ void __launch_bounds__(256) yolo_pool_select_kernel(const __grid_constant__ YoloParams p, ImgState* __restrict__ states,
                                                               unsigned* __restrict__ hist, int* __restrict__ flags) {
    const int img = blockIdx.x;
    ImgState st = states[img];
    if (st.phase != PHASE_POOL) return;
    __shared__ unsigned s_part[256];
    __shared__ unsigned s_h[kBins];
    const int nb = 1 << level_bits(st.level);
    load_hist_desc(hist + (size_t)img * kBins, nb, s_h, s_part);
    if (threadIdx.x != 0) return;
    if (st.level == 0) {
        st.cap = band_cap(p, st);
        st.above = 0;
        st.prefix = 0;
    }
    const long long scale = st.sampled ? p.hist_stride : 1;
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    const long long want = st.sampled ? 2ll * st.cap : (long long)st.cap - st.above;  // > 0
    long long cum = 0;
    int b = -1;
    for (int t = 0; t < 256 && b < 0; ++t) {
        if ((cum + s_part[t]) * scale < want) { cum += s_part[t]; continue; }
        for (int j = 0; j < kBins / 256; ++j) {
            const int slot = t * (kBins / 256) + j;
            if ((cum + s_h[slot]) * scale >= want) { b = nb - 1 - slot; break; }
            cum += s_h[slot];
        }
    }
    const unsigned long long base = st.level == 0 ? 0ull : (st.prefix << (shift + bits));
    long long count;
    if (b < 0) {
        // everything that is left (under this prefix) is fewer than wanted: take all of it
        st.pool_lo = base;
        count = st.above + cum * scale;
    } else {
        const long long incl = st.above + (cum + s_h[nb - 1 - b]) * scale;
        long long fits = st.sampled ? incl + incl / 2 : incl;
        const long long all = (long long)p.total_ca * p.classes;  // an image has no more candidates than this, whatever the estimate says
        if (fits > all) fits = all;
        if (fits <= p.pool_max || (!st.sampled && st.level == kLevels - 1)) {
            st.pool_lo = base + ((unsigned long long)b << shift);
            count = incl;
        } else {
            if (st.sampled) st.sampled = 0;  // same level again, every block this time
            else {
                st.above += (int)cum;
                st.prefix = (st.level == 0 ? 0ull : (st.prefix << bits)) | (unsigned long long)b;
                st.level += 1;
            }
            atomicAdd(&flags[FLAG_POOL_PENDING], 1);
            states[img] = st;
            return;
        }
    }
    st.phase = PHASE_FILL;
    st.direct = (st.sampled ? count + count / 2 : count) <= p.band_max ? 1 : 0;
    if (st.direct) {
        st.lo = st.pool_lo;
        st.band_count = (int)count;
        st.exhausted = 1;
    }
    st.pool_count = 0;
    states[img] = st;
}

// After the fill pass: a filled pool goes to band selection, a directly filled band to NMS.  A fill that found more
// keys than its destination holds (possible only after a sampled histogram) is thrown away and the image starts over
// with the full histogram.
__global__ void yolo_after_fill_kernel(ImgState* __restrict__ states, int* __restrict__ band_fill, int* __restrict__ pool_fill, int batch,
                                       int band_max, int pool_max, int hist_stride, int* __restrict__ flags,
                                       unsigned long long* __restrict__ key_and_or) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch || states[i].phase != PHASE_FILL) return;
    int* fill = states[i].direct ? band_fill + i : pool_fill + i;
    const int n = *fill;
    if (n > (states[i].direct ? band_max : pool_max)) {
        *fill = 0;
        key_and_or[2 * i] = ~0ull;
        key_and_or[2 * i + 1] = 0ull;
        states[i].phase = PHASE_POOL;
        states[i].sampled = 0;
        states[i].level = 0;
        atomicAdd(&flags[FLAG_POOL_PENDING], 1);
        return;
    }
    states[i].sampled = hist_stride > 1 ? 1 : 0;  // for the next pool of this image
    const unsigned long long k_and = key_and_or[2 * i], k_or = key_and_or[2 * i + 1];
    key_and_or[2 * i] = ~0ull;
    key_and_or[2 * i + 1] = 0ull;
    if (states[i].direct) {
        states[i].band_count = n;
        states[i].phase = PHASE_BAND;
    } else {
        // digits on which the AND and the OR of the pool's keys agree are shared by all of them: the selection starts below them
        int level = 0;
        unsigned long long prefix = 0ull;
        const unsigned long long diff = k_and ^ k_or;
        while (n > 0 && level < kLevels - 1) {
            const int sh = level_shift(level), bt = level_bits(level);
            const unsigned long long m = ((1ull << bt) - 1ull) << sh;
            if (diff & m) break;
            prefix = (prefix << bt) | ((k_and & m) >> sh);
            ++level;
        }
        states[i].pool_count = n;
        states[i].phase = PHASE_SELECT;
        states[i].level = states[i].start_level = level;
        states[i].prefix = states[i].start_prefix = prefix;
        states[i].fresh = 1;
    }
}

// Passes over the pool: one thread per two keys; integer work only.
// MODE 0: histogram of digit `level` under `prefix` of the unconsumed keys, plus the AND and OR of those keys (they tell
// the selection which further digits all of them share).  Lanes of a warp that fall into the same bin are merged into one
// shared-memory add.  MODE 1: collect the keys of the band [lo, hi).
template <int MODE>
__global__ void __launch_bounds__(256) yolo_pool_scan_kernel(const __grid_constant__ YoloParams p, const ImgState* __restrict__ states,
                                                             unsigned* __restrict__ hist, unsigned long long* __restrict__ key_and_or,
                                                             unsigned long long* __restrict__ band, int* __restrict__ band_fill,
                                                             const unsigned long long* __restrict__ pool) {
    const int img = blockIdx.y;
    const ImgState st = states[img];
    if (st.phase != (MODE == 0 ? PHASE_SELECT : PHASE_BAND) || (MODE == 1 && st.direct)) return;
    const unsigned n = (unsigned)st.pool_count;
    const unsigned chunk_begin = blockIdx.x * kPoolChunk;
    if (chunk_begin >= n) return;
    __shared__ unsigned s_hist[MODE == 0 ? kBins : 1];
    __shared__ unsigned long long s_and, s_or;
    if (MODE == 0) {
        for (int i = threadIdx.x; i < kBins; i += blockDim.x) s_hist[i] = 0;
        if (threadIdx.x == 0) { s_and = ~0ull; s_or = 0ull; }
        __syncthreads();
    }
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    const unsigned long long* img_pool = pool + (size_t)img * p.pool_max;
    unsigned long long t_and = ~0ull, t_or = 0ull;
    for (unsigned base = chunk_begin; base < chunk_begin + kPoolChunk && base < n; base += 2u * blockDim.x) {  // uniform trip count
        const unsigned i0 = base + 2u * threadIdx.x;
        ulonglong2 v = make_ulonglong2(0ull, 0ull);
        if (i0 + 1 < n) v = *reinterpret_cast<const ulonglong2*>(img_pool + i0);
        else if (i0 < n) v.x = img_pool[i0];
        const unsigned long long ks[2] = {v.x, v.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const unsigned long long key = ks[e];
            bool valid = i0 + e < n && key < st.hi;
            if (MODE == 0) {
                valid = valid && (st.level == 0 || (key >> (shift + bits)) == st.prefix);
                unsigned bin = 0xFFFFFFFFu;
                if (valid) {
                    bin = (unsigned)(key >> shift) & ((1u << bits) - 1u);
                    t_and &= key;
                    t_or |= key;
                }
                const unsigned same = __match_any_sync(0xffffffffu, bin);
                if (valid && (threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&s_hist[bin], (unsigned)__popc(same));
            } else if (valid && key >= st.lo) {
                const int slot = atomicAdd(&band_fill[img], 1);
                if (slot < p.band_max) band[(size_t)img * p.band_max + slot] = key;
            }
        }
    }
    if (MODE == 0) {
        for (int o = 16; o > 0; o >>= 1) {
            t_and &= __shfl_xor_sync(0xffffffffu, t_and, o);
            t_or |= __shfl_xor_sync(0xffffffffu, t_or, o);
        }
        if ((threadIdx.x & 31) == 0) { atomicAnd(&s_and, t_and); atomicOr(&s_or, t_or); }
        __syncthreads();
        for (int b = threadIdx.x; b < kBins; b += blockDim.x)
            if (s_hist[b]) atomicAdd(&hist[(size_t)img * kBins + b], s_hist[b]);
        if (threadIdx.x == 0) { atomicAnd(&key_and_or[2 * img], s_and); atomicOr(&key_and_or[2 * img + 1], s_or); }
    }
}

// One block per image: walk the digit histogram of the pool from the top, either fix the band's lower bound or descend
// into the digit that holds too many candidates (skipping the digits all keys under it share).  Leaves the histogram zeroed.
__global__ void __launch_bounds__(256) yolo_select_kernel(const __grid_constant__ YoloParams p, ImgState* __restrict__ states,
                                                          unsigned* __restrict__ hist, unsigned long long* __restrict__ key_and_or,
                                                          int* __restrict__ flags) {
    const int img = blockIdx.x;
    ImgState st = states[img];
    if (st.phase != PHASE_SELECT) return;
    __shared__ unsigned s_part[256];
    __shared__ unsigned s_h[kBins];
    const int nb = 1 << level_bits(st.level);
    const int per = kBins / 256;
    load_hist_desc(hist + (size_t)img * kBins, nb, s_h, s_part);
    if (threadIdx.x != 0) return;
    const unsigned long long k_and = key_and_or[2 * img], k_or = key_and_or[2 * img + 1];
    key_and_or[2 * img] = ~0ull;
    key_and_or[2 * img + 1] = 0ull;
    // ---- one thread decides (a few hundred steps at most)
    if (st.fresh) {  // first pass of this band: level and prefix are the pool's starting point
        st.cap = band_cap(p, st);
        st.above = 0;
        st.fresh = 0;
    }
    const unsigned cap_left = (unsigned)(st.cap - st.above);
    const int shift = level_shift(st.level), bits = level_bits(st.level);
    unsigned cum = 0, everything = 0;
    int owner = -1;
    for (int t = 0; t < 256; ++t) everything += s_part[t];
    for (int t = 0; t < 256; ++t) {
        if (cum + s_part[t] > cap_left) { owner = t; break; }
        cum += s_part[t];
    }
    if (owner < 0) {
        // everything that is left of the pool (under this prefix) fits into the band
        const bool whole_pool = st.level == st.start_level;  // nothing was cut off above this level: the rest of the pool is the band
        st.lo = whole_pool ? st.pool_lo : (st.prefix << (shift + bits));
        st.band_count = st.above + (int)cum;
        st.exhausted = whole_pool ? 1 : 0;
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
        if (s_h[nb - 1 - b] == everything) {
            // every key of this pass sits in bin b: digits on which their AND and OR agree are shared by all of them
            const unsigned long long diff = k_and ^ k_or;
            while (st.level < kLevels - 1) {
                const int sh = level_shift(st.level), bt = level_bits(st.level);
                const unsigned long long m = ((1ull << bt) - 1ull) << sh;
                if (diff & m) break;
                st.prefix = (st.prefix << bt) | ((k_and & m) >> sh);
                st.level += 1;
            }
        }
        atomicAdd(&flags[FLAG_SELECT_PENDING], 1);
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
                                                           ln_detection* __restrict__ records, int* __restrict__ flags) {
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
            // the mask row of candidate i + 1 is fetched while candidate i is decided: the loop is a chain of dependent steps and
            // the shared-memory latency would otherwise sit on it
            unsigned row = lane < 16 ? mask[lane] : 0u;
            for (int i = 0; i < m && kept_now < p.k_eff; ++i) {
                const unsigned next = (lane < 16 && i + 1 < m) ? mask[(i + 1) * 16 + lane] : 0u;
                const unsigned r = __shfl_sync(0xffffffffu, removed, i >> 5);
                if (!((r >> (i & 31)) & 1u)) {
                    removed |= row;
                    if (lane == 0) cpos[i] = kept_now;
                    ++kept_now;
                }
                row = next;
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
        if (st.kept >= p.k_eff || (st.exhausted && st.pool_lo == 0ull)) st.phase = PHASE_DONE;
        else {
            atomicAdd(&flags[FLAG_ACTIVE], 1);
            st.level = 0;
            if (st.exhausted) {  // the pool is used up: the next one starts below it
                st.phase = PHASE_POOL;
                st.prefix = 0;
                st.above = 0;
                atomicAdd(&flags[FLAG_NEED_POOL], 1);
            } else {
                st.phase = PHASE_SELECT;
                st.level = st.start_level;
                st.prefix = st.start_prefix;
                st.fresh = 1;
            }
        }
        states[img] = st;
    }
}

__global__ void yolo_init_states_kernel(ImgState* states, unsigned long long* key_and_or, const int* img_w, const int* img_h, int batch, int hist_stride) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch) return;
    ImgState s;
    s.hi = ~0ull; s.lo = 0; s.prefix = 0; s.pool_lo = 0;
    s.level = 0; s.phase = PHASE_POOL; s.cap = 0; s.above = 0; s.band_count = 0; s.kept = 0; s.exhausted = 0;
    s.img_w = img_w[i]; s.img_h = img_h[i]; s.last_gain = -1; s.direct = 0; s.pool_count = 0; s.sampled = hist_stride > 1 ? 1 : 0;
    s.start_level = 0; s.fresh = 1; s.start_prefix = 0;
    states[i] = s;
    key_and_or[2 * i] = ~0ull;
    key_and_or[2 * i + 1] = 0ull;
}

__global__ void yolo_counts_kernel(const ImgState* states, int* counts, int batch, int max_per_image) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < batch) counts[i] = states[i].kept < max_per_image ? states[i].kept : max_per_image;
}

// Largest distance between the approximate and the exact confidence key over a sweep of logits (debug aid that
// justifies kKeySlack): objectness sweeps [obj_lo, obj_hi], class logit sweeps [x_lo, x_hi].
__global__ void yolo_key_error_kernel(float obj_lo, float obj_hi, float x_lo, float x_hi, int n_obj, int n_x, unsigned* __restrict__ worst) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_obj * n_x) return;
    const int io = i / n_x, ix = i - io * n_x;
    const float o = obj_lo + (obj_hi - obj_lo) * ((float)io / (float)(n_obj > 1 ? n_obj - 1 : 1));
    const float x = x_lo + (x_hi - x_lo) * ((float)ix / (float)(n_x > 1 ? n_x - 1 : 1));
    const float obj = ln_det_sigmoid(o);
    unsigned klo, khi;
    approx_score_key(obj, x, klo, khi);
    const unsigned mid = klo + (khi - klo) / 2u;
    const unsigned exact = conf_key(__fmul_rn(obj, ln_det_sigmoid(x)));
    const unsigned d = mid > exact ? mid - exact : exact - mid;
    atomicMax(worst, d);
}

// ---- decode only (parity helper): per (anchor, cell) counts, then ordered writes ---------------
__global__ void yolo_decode_count_kernel(const __grid_constant__ YoloParams p, int img, int* __restrict__ counts) {
    const int ca = blockIdx.x * blockDim.x + threadIdx.x;
    if (ca >= p.total_ca) return;
    const HeadDev& h = p.heads[find_head(p, ca)];
    const int stride = h.gw * h.gh, epa = h.classes + 5;
    const int local = ca - h.ca_base, a = local / stride, idx = local - a * stride;
    const float* img_raw = h.raw + (size_t)img * h.n_anchor * epa * stride;
    const float obj = score_obj(h, img_raw[(size_t)(a * epa + 4) * stride + idx]);
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
    const float obj = score_obj(h, img_raw[(size_t)(a * epa + 4) * stride + idx]);
    const float obj_reported = head_act(img_raw[(size_t)(a * epa + 4) * stride + idx], h.new_coords);
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
            d.class_id = (float)c; d.confidence = conf; d.objectness = obj_reported; d.x = b.x; d.y = b.y; d.w = b.w; d.h = b.h;
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
        if (s.kind < 0 || s.kind > 2) return ln_fail(ctx, LN_ERR_ARG, "%s: head %d has kind %d (0 = yolo, 1 = yolox, 2 = predecoded distribution head)", who, k, s.kind);
        if (s.kind != 0 && s.n_anchor != 1) return ln_fail(ctx, LN_ERR_ARG, "%s: head %d is anchor-free and takes n_anchor = 1", who, k);
        h.gw = (int)s.raw->w; h.gh = (int)s.raw->h; h.classes = s.classes; h.n_anchor = s.n_anchor;
        h.kind = s.kind;
        h.new_coords = s.kind != 0 ? 1 : s.new_coords;  // the modern heads hold probabilities already
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

struct Scratch {
    size_t sz_states, sz_hist, sz_band, sz_fill, sz_kbox, sz_kcls, sz_rec, sz_dims, sz_cnt, sz_andor, sz_flags, sz_pool, total;
};

// Sizes of the working arrays of one call.  pool_entries = 0 picks the pool size: every candidate of an image when that
// keeps the pools of the call within kPoolBytesTarget, otherwise that budget split over the images (at least 65536 keys).
void scratch_layout(YoloParams* p, int pool_entries, Scratch* s) {
    const int64_t B = p->batch;
    const int64_t per_image = (int64_t)p->total_ca * p->classes;
    int64_t pm = pool_entries;
    if (pm <= 0) {
        pm = kPoolBytesTarget / 8 / B;
        if (pm < 65536) pm = 65536;
    }
    if (pm > per_image) pm = per_image;
    if (pm < p->band_max + 1) pm = p->band_max + 1;  // a pool is only used for more than a band holds
    pm = ln_round_up(pm, 2);                         // 16-byte rows
    p->pool_max = (int)pm;
    // sampling pays once an image has many blocks of slots; small images are histogrammed in full
    p->hist_stride = (p->total_ca + 255) / 256 >= 64 ? 8 : 1;
    s->sz_states = (size_t)ln_round_up(B * (int64_t)sizeof(ImgState), 256);
    s->sz_hist = (size_t)B * kBins * 4;
    s->sz_band = (size_t)B * p->band_max * 8;
    s->sz_fill = (size_t)ln_round_up(B * 8, 256);  // band_fill, pool_fill
    s->sz_kbox = (size_t)B * p->k_eff * sizeof(float4);
    s->sz_kcls = (size_t)ln_round_up(B * p->k_eff * 4, 256);
    s->sz_rec = (size_t)ln_round_up(B * p->max_per_image * (int64_t)sizeof(ln_detection), 256);
    s->sz_dims = (size_t)ln_round_up(B * 8, 256);
    s->sz_cnt = (size_t)ln_round_up(B * 4, 256);
    s->sz_andor = (size_t)ln_round_up(B * 16, 256);
    s->sz_flags = 256;
    s->sz_pool = (size_t)B * (size_t)pm * 8;
    s->total = s->sz_states + s->sz_hist + s->sz_band + s->sz_fill + s->sz_kbox + s->sz_kcls + s->sz_rec + s->sz_dims + s->sz_cnt + s->sz_andor +
               s->sz_flags + s->sz_pool;
}

int check_options(ln_ctx* ctx, YoloParams* p, const ln_detect_options* opts, const int32_t* image_w, const int32_t* image_h, int band_max, const char* who) {
    p->thr = opts->confidence_threshold;
    // apply_nms returns at once for a threshold <= 0 (detect.rs:1449-1452): nothing is suppressed.  The kernels test
    // `iou > nms_thr`, which no IoU passes when the threshold is +infinity.
    p->nms_thr = opts->nms_threshold > 0.0f ? opts->nms_threshold : INFINITY;
    p->letterbox = opts->letterbox;
    p->max_per_image = opts->max_per_image;
    p->k_eff = opts->top_k > 0 && opts->top_k < opts->max_per_image ? opts->top_k : opts->max_per_image;
    p->band_max = band_max ? band_max : (p->k_eff <= 1024 ? kBandMaxLarge : kBandMaxSmall);
    if (p->k_eff > 4096) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "%s: at most 4096 detections per image (top_k / max_per_image)", who);
    for (int i = 0; i < p->batch; ++i)
        if (image_w[i] <= 0 || image_h[i] <= 0) return ln_fail(ctx, LN_ERR_ARG, "image dimensions must be positive for network detection decoding");
    return LN_OK;
}

// The whole decode + NMS call over working memory that the caller provides (s.total bytes at `scratch`, 256-byte aligned).
int run_decode_nms(ln_ctx* ctx, const YoloParams& p, const Scratch& s, unsigned char* scratch, const int32_t* image_w, const int32_t* image_h,
                   ln_detection* records_host, int32_t* counts_host, const char* who, void* pinned_stage = nullptr) {
    const int B = p.batch;
    unsigned char* q = scratch;
    ImgState* states = (ImgState*)q; q += s.sz_states;
    unsigned* hist = (unsigned*)q; q += s.sz_hist;
    unsigned long long* band = (unsigned long long*)q; q += s.sz_band;
    int* band_fill = (int*)q; int* pool_fill = band_fill + B; q += s.sz_fill;
    float4* kept_box = (float4*)q; q += s.sz_kbox;
    int* kept_cls = (int*)q; q += s.sz_kcls;
    ln_detection* records = (ln_detection*)q; q += s.sz_rec;
    int* dims = (int*)q; q += s.sz_dims;
    int* counts = (int*)q; q += s.sz_cnt;
    unsigned long long* key_and_or = (unsigned long long*)q; q += s.sz_andor;
    int* flags = (int*)q; q += s.sz_flags;
    unsigned long long* pool = (unsigned long long*)q;
#define LN_Y(call)                                                                                     \
    do {                                                                                               \
        cudaError_t e__ = (call);                                                                      \
        if (e__ != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "%s: %s: %s", who, #call, cudaGetErrorString(e__)); \
    } while (0)
    const bool dbg = getenv("LN_DEBUG_NMS") != nullptr;
    auto now = []() { timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts); return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6; };
    const double t_begin = dbg ? now() : 0;
    // the working memory keeps whatever an earlier call left: clear everything the kernels expect to start at zero
    LN_Y(cudaMemsetAsync(hist, 0, s.sz_hist, ctx->stream));
    LN_Y(cudaMemsetAsync(band_fill, 0, s.sz_fill, ctx->stream));
    LN_Y(cudaMemsetAsync(flags, 0, s.sz_flags, ctx->stream));
    LN_Y(cudaMemcpyAsync(dims, image_w, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    LN_Y(cudaMemcpyAsync(dims + B, image_h, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    yolo_init_states_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(states, key_and_or, dims, dims + B, B, p.hist_stride);
    ctx->launches++;

    const size_t nms_smem = (size_t)p.band_max * 8 + (size_t)(p.k_eff + kChunk) * sizeof(float4) + (size_t)kChunk * (kChunk / 32) * 4 +
                            (size_t)(p.k_eff + kChunk) * 4 + (size_t)kChunk * 8 + 64;
    LN_Y(cudaFuncSetAttribute(yolo_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)nms_smem));
    const dim3 scan_grid((p.total_ca + 255) / 256, B);
    const dim3 pool_grid((unsigned)((p.pool_max + kPoolChunk - 1) / kPoolChunk), B);
    int* h_flags = ctx->h_status + 4;  // 4 ints
    const int max_rounds = 4096;
    // with LN_DEBUG_NMS set, every kernel is followed by a synchronize and its wall time is added to its class
    double t_k[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    double t_mark = 0;
    auto tick = [&]() { if (dbg) { cudaStreamSynchronize(ctx->stream); t_mark = now(); } };
    auto tock = [&](int k) { if (dbg) { cudaStreamSynchronize(ctx->stream); t_k[k] += now() - t_mark; } };
    int n_full = 0, n_pool_passes = 0, round = 0;
    bool need_pool = true;
    for (; round < max_rounds; ++round) {
        // selection: pools for the images that need one, then a band inside every pool; repeated while some image descends a digit
        for (int step = 0; step < 2 * kLevels + 2; ++step) {
            if (need_pool) {
                tick();
                yolo_head_hist_kernel<<<scan_grid, 256, 0, ctx->stream>>>(p, states, hist);
                tock(0); tick();
                yolo_pool_select_kernel<<<B, 256, 0, ctx->stream>>>(p, states, hist, flags);
                tock(1); tick();
                yolo_head_fill_kernel<<<scan_grid, 256, 0, ctx->stream>>>(p, states, band, band_fill, pool, pool_fill, key_and_or);
                tock(2);
                yolo_after_fill_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(states, band_fill, pool_fill, B, p.band_max, p.pool_max, p.hist_stride, flags, key_and_or);
                ctx->launches += 4;
                n_full += 2;
            }
            tick();
            yolo_pool_scan_kernel<0><<<pool_grid, 256, 0, ctx->stream>>>(p, states, hist, key_and_or, band, band_fill, pool);
            tock(3); tick();
            yolo_select_kernel<<<B, 256, 0, ctx->stream>>>(p, states, hist, key_and_or, flags);
            tock(4);
            ctx->launches += 2;
            ++n_pool_passes;
            LN_Y(cudaMemcpyAsync(h_flags, flags, 16, cudaMemcpyDeviceToHost, ctx->stream));
            LN_Y(cudaMemsetAsync(flags, 0, 16, ctx->stream));
            LN_Y(cudaStreamSynchronize(ctx->stream));
            need_pool = h_flags[FLAG_POOL_PENDING] != 0;
            if (!need_pool && h_flags[FLAG_SELECT_PENDING] == 0) break;
        }
        tick();
        yolo_pool_scan_kernel<1><<<pool_grid, 256, 0, ctx->stream>>>(p, states, hist, key_and_or, band, band_fill, pool);
        tock(5); tick();
        yolo_nms_kernel<<<B, 1024, nms_smem, ctx->stream>>>(p, states, band, band_fill, kept_box, kept_cls, records, flags);
        tock(6);
        ctx->launches += 2;
        LN_Y(cudaMemcpyAsync(h_flags, flags, 16, cudaMemcpyDeviceToHost, ctx->stream));
        LN_Y(cudaMemsetAsync(flags, 0, 16, ctx->stream));
        LN_Y(cudaMemsetAsync(pool_fill, 0, (size_t)B * 4, ctx->stream));
        LN_Y(cudaStreamSynchronize(ctx->stream));
        if (h_flags[FLAG_ACTIVE] == 0) break;
        need_pool = need_pool || h_flags[FLAG_NEED_POOL] != 0;
    }
    const double t_loop = dbg ? now() : 0;
    if (dbg) fprintf(stderr, "[ln_yolo] batch %d: %d rounds, %d passes over the heads, %d pool passes; ms: head histogram %.3f, pool select %.3f, head fill %.3f, "
                     "pool histogram %.3f, band select %.3f, band collect %.3f, sort + nms %.3f; band_max %d, pool_max %d, k_eff %d\n",
                     B, round + 1, n_full, n_pool_passes, t_k[0], t_k[1], t_k[2], t_k[3], t_k[4], t_k[5], t_k[6], p.band_max, p.pool_max, p.k_eff);
    if (round == max_rounds) return ln_fail(ctx, LN_ERR_TIMEOUT, "%s: NMS did not finish in %d rounds", who, max_rounds);
    yolo_counts_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(states, counts, B, p.max_per_image);
    ctx->launches++;
    LN_Y(cudaGetLastError());
    const size_t rec_bytes = (size_t)B * p.max_per_image * sizeof(ln_detection);
    // a caller that passes page-locked buffers gets its records by DMA, without the staging copy below
    if (pinned_stage) {
        cudaPointerAttributes pa_r, pa_c;
        if (cudaPointerGetAttributes(&pa_r, records_host) == cudaSuccess && cudaPointerGetAttributes(&pa_c, counts_host) == cudaSuccess &&
            pa_r.type == cudaMemoryTypeHost && pa_c.type == cudaMemoryTypeHost)
            pinned_stage = nullptr;
        (void)cudaGetLastError();  // (an unregistered pointer is not an error here)
    }
    if (pinned_stage) {
        // through pinned memory: the copy runs at link speed instead of being staged page by page by the driver
        LN_Y(cudaMemcpyAsync(pinned_stage, records, rec_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        LN_Y(cudaMemcpyAsync((unsigned char*)pinned_stage + rec_bytes, counts, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
        LN_Y(cudaStreamSynchronize(ctx->stream));
        memcpy(records_host, pinned_stage, rec_bytes);
        memcpy(counts_host, (unsigned char*)pinned_stage + rec_bytes, (size_t)B * 4);
    } else {
        LN_Y(cudaMemcpyAsync(counts_host, counts, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
        LN_Y(cudaMemcpyAsync(records_host, records, rec_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        LN_Y(cudaStreamSynchronize(ctx->stream));
    }
    if (dbg) fprintf(stderr, "[ln_yolo] whole call %.3f ms, of which the read-back of counts and records %.3f ms\n", now() - t_begin, now() - t_loop);
#undef LN_Y
    return LN_OK;
}

}  // namespace

extern "C" {

int32_t ln_yolo_decode_nms(ln_ctx* ctx, const ln_yolo_head* heads, int32_t n_heads, int32_t net_w, int32_t net_h, const int32_t* image_w,
                           const int32_t* image_h, const ln_detect_options* opts, ln_detection* records_host, int32_t* counts_host) {
    const char* who = "ln_yolo_decode_nms";
    if (!ctx || !heads || !image_w || !image_h || !opts || !records_host || !counts_host) return ln_fail(ctx, LN_ERR_ARG, "%s: NULL argument", who);
    if (opts->max_per_image < 1) return ln_fail(ctx, LN_ERR_ARG, "%s: max_per_image must be positive", who);
    YoloParams p;
    int rc = fill_params(ctx, &p, heads, n_heads, net_w, net_h, who);
    if (rc) return rc;
    rc = check_options(ctx, &p, opts, image_w, image_h, 0, who);
    if (rc) return rc;
    Scratch s;
    scratch_layout(&p, ctx->nms_pool_entries, &s);
    cudaSetDevice(ctx->device);
    unsigned char* scratch = (unsigned char*)ln_pool_alloc(ctx, s.total);
    if (!scratch) return LN_ERR_CUDA;
    const size_t stage_bytes = (size_t)p.batch * p.max_per_image * sizeof(ln_detection) + (size_t)p.batch * 4;
    if (ctx->h_stage_bytes < stage_bytes) {
        if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
        ctx->h_stage = nullptr;
        ctx->h_stage_bytes = 0;
        if (cudaMallocHost(&ctx->h_stage, stage_bytes) == cudaSuccess) ctx->h_stage_bytes = stage_bytes;
        else { ctx->h_stage = nullptr; cudaGetLastError(); }  // no pinned memory to be had: read back directly
    }
    rc = run_decode_nms(ctx, p, s, scratch, image_w, image_h, records_host, counts_host, who, ctx->h_stage);
    ln_pool_free(ctx, scratch, s.total);
    return rc;
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
    rc = check_options(ctx, &p, opts, image_w, image_h, kBandMaxSmall, who);
    if (rc) return rc;
    // the pool gets what the fixed array has left after the other working arrays, and must hold every candidate of an
    // image: this entry point never takes the extra passes a smaller pool can need
    Scratch s;
    scratch_layout(&p, 0, &s);
    const int64_t per_image = (int64_t)p.total_ca * p.classes;
    if (p.pool_max < per_image || s.total > (size_t)LN_NOALLOC_SCRATCH_BYTES)
        return ln_fail(ctx, LN_ERR_UNSUPPORTED,
                       "%s: this call needs %zu bytes of working memory (batch %d, %lld candidates per image, %d records per image) but the fixed "
                       "array holds %u; use a smaller batch, fewer records, or ln_yolo_decode_nms",
                       who, s.total - s.sz_pool + (size_t)p.batch * (size_t)ln_round_up(per_image, 2) * 8, p.batch, (long long)per_image, p.max_per_image,
                       LN_NOALLOC_SCRATCH_BYTES);
    cudaSetDevice(ctx->device);
    if (!g_noalloc_ptr[ctx->device]) {
        // once per device, with that device current: the address of the module's array on this device
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, ln_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return ln_fail(ctx, LN_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", who, cudaGetErrorString(e));
        g_noalloc_ptr[ctx->device] = (unsigned char*)ptr;
    }
    return run_decode_nms(ctx, p, s, g_noalloc_ptr[ctx->device], image_w, image_h, records_host, counts_host, who);
}

// Debug aid: largest distance (in confidence-key units) between the approximate and the exact score over a sweep.
int32_t ln_debug_score_key_error(ln_ctx* ctx, float obj_lo, float obj_hi, float x_lo, float x_hi, int32_t n_obj, int32_t n_x, uint32_t* worst) {
    if (!ctx || !worst || n_obj < 1 || n_x < 1) return ln_fail(ctx, LN_ERR_ARG, "ln_debug_score_key_error: bad argument");
    cudaSetDevice(ctx->device);
    unsigned* d = (unsigned*)ln_pool_alloc(ctx, 256);
    if (!d) return LN_ERR_CUDA;
    cudaMemsetAsync(d, 0, 4, ctx->stream);
    const long long total = (long long)n_obj * n_x;
    yolo_key_error_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(obj_lo, obj_hi, x_lo, x_hi, n_obj, n_x, d);
    ctx->launches++;
    cudaError_t e = cudaMemcpyAsync(worst, d, 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    ln_pool_free(ctx, d, 256);
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "ln_debug_score_key_error: %s", cudaGetErrorString(e));
    return LN_OK;
}

int32_t ln_ctx_set_nms_pool_entries(ln_ctx* ctx, int64_t entries) {
    if (!ctx || entries < 0 || entries > (1ll << 30)) return ln_fail(ctx, LN_ERR_ARG, "ln_ctx_set_nms_pool_entries: entries must be in [0, 2^30]");
    ctx->nms_pool_entries = (int)entries;
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
