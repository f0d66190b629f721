// ops.cu -- the Conv / Gemm / MatMul operators over the implicit-GEMM kernel: descriptor
// parsing and validation, path selection, the drop-in eval entry points and the prepared
// (device-resident) path.  Public view: include/one_cuda.h.
//
// Reference behaviour mirrored here (device/x86/Conv/conv.c:13-66):
//   * a Conv without bias gets NO activation (the reference returns before do_act, :18-27);
//   * dilations are carried in the config but ignored by every reference kernel, so they are
//     ignored here as well;
//   * the int8 path pads all four sides by pads[0] (:979-999); unequal pads are rejected;
//   * group != 1 is treated as depthwise, as the reference does; it runs a CUDA-core kernel on the
//     reference layout (fp32 and int8).
// Two deliberate differences.  The reference's im2col indexes with out_h*out_h (:189-190) and is
// only right for square outputs; non-square outputs are computed correctly here.  And with unequal
// strides the reference disagrees with itself: its kernels step along w by strides[0] and along h by
// strides[1] (conv.c:186-187), while its shape inference divides H by strides[0] and W by strides[1]
// (host/ops/conv.h:44-47).  Here both follow the kernels (strides[0] along w), so a y descriptor written
// by the reference's host for unequal strides is refused with ONE_ERR_BAD_SHAPE rather than filled with
// a tensor of another shape; equal strides, the only case the reference's models use, are unaffected.
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/one_cuda.h"
#include "ctx.h"
#include "glue.cuh"
#include "igemm.cuh"
#include "sm100_prims.cuh"

using namespace one;

namespace {

thread_local int t_eval_prec = ONE_PREC_TF32;
thread_local int t_tile_n = 0;
static std::atomic<int> g_cta_pairs{1};   // tile codes 1xxx (pairs of CTAs) are accepted
static std::atomic<int> g_half_tiles{1};  // tile codes 2xxx (two 128-row halves per CTA) are accepted
static std::atomic<int> g_wide_epi{1};    // tile codes 4xxx (twelve epilogue warps) are accepted
thread_local int t_pairing = 1;      // width pairing of narrow multi-tap convolutions (see pair_geometry)
thread_local int t_last_split = 1;   // K ranges the last contraction enqueued by this thread was cut into
thread_local int t_split_k = 0;   // 0: the library's choice, 1: never split, n > 1: force n ranges (clamped to the K blocks)

struct ConvGeom {
    int N, C, H, W, OC, KH, KW, OH, OW, sw, sh, pt, pl, pb, pr;
    int depthwise;   // group != 1: one input channel per output channel (the reference's reading of any group)
};
struct ConvEpi {
    int has_bias, act, int8;
    float p0, p1, in_scale;
};
enum ConvPath { PATH_TILED = 0, PATH_IM2COL = 1, PATH_EXPLICIT = 2, PATH_S2D = 3, PATH_PATCH = 4 };
struct ConvPlan {
    int kind, es, adt;        // MMA kind, element size, activation DType
    int path;
    int w_pitch;              // elements per packed weight row (>= K)
    int slab_bytes, slab_elems, num_kb, c_slabs, bn;
    int cta2;                 // launch as pairs of CTAs sharing 256-row tiles (tile codes 1xxx)
    int mh;                   // 128-row halves per CTA tile: 1, or 2 (tile codes 2xxx)
    int nw;                   // epilogue warps: 8, or 12 (tile codes 4xxx)
    // PATH_S2D: the stride-2 conv re-expressed as a stride-1 conv over the space-to-depth image;
    // bw = columns carried per position (2, or 4: neighbouring positions overlap and one filter
    // position covers 4 taps along w, placed dil_w = bw / 2 positions apart)
    int eh, ew, Hs, Ws, Cp, KH2, KW2, pt2, pl2, pb2, pr2, bw, dil_w;
};
inline bool reads_reference_layout(const ConvPlan &p) { return p.path == PATH_EXPLICIT || p.path == PATH_S2D || p.path == PATH_PATCH; }

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
// A tile choice is a code: the output-tile width (64 / 128 / 192 / 256), plus 1000 when the launch runs as
// pairs of CTAs that share 256-row tiles (widths 128 / 192 / 256 only), plus 2000 when every CTA takes
// 256-row tiles as two 128-row halves against one tile of B (widths 64 / 128 only), or plus 4000 when the CTA
// runs twelve epilogue warps (three groups) behind a shallower operand ring (widths 64 / 128 only).
inline int tile_bn(int code) { return code % 1000; }
inline bool tile_cta2(int code) { return code >= 1000 && code < 2000; }
inline int tile_mh(int code) { return code >= 2000 && code < 3000 ? 2 : 1; }
inline int tile_nw(int code) { return code >= 4000 && code < 5000 ? 12 : 8; }
inline bool valid_tile(int code)
{
    const int bn = tile_bn(code);
    if (bn != 64 && bn != 128 && bn != 192 && bn != 256) return false;
    return code < 1000 || (code < 2000 && bn != 64) || (code >= 2000 && code < 3000 && bn <= 128) || (code >= 4000 && code < 5000 && bn <= 128);
}
// Tile width: as wide as the output allows (A is then re-read fewer times), narrowed while the
// launch would leave SMs without a tile.
inline int pick_bn(int n, long long m = 1 << 30)
{
    if (valid_tile(t_tile_n)) return t_tile_n;
    int bn = n <= 64 ? 64 : (n <= 128 ? 128 : 256);
    // widths that are multiples of 192 but not of 256 (ViT-Tiny: 192, 576, 768) waste a quarter of a
    // 256-wide tile; a 192-wide tile fits them exactly
    if (n % 192 == 0 && n % 256 != 0 && m * (n / 192) >= 148 * 128LL) return 192;
    const long long m_tiles = (m + 127) / 128;
    while (bn > 64 && m_tiles * ((n + bn - 1) / bn) < 148) bn >>= 1;
    return bn;
}
inline bool kind_is_16(int kind) { return kind == KIND_BF16 || kind == KIND_F16; }
inline int kind_es(int kind) { return kind == KIND_TF32 ? 4 : (kind_is_16(kind) ? 2 : 1); }
inline int kind_dt(int kind) { return kind == KIND_TF32 ? DT_F32 : (kind == KIND_BF16 ? DT_BF16 : (kind == KIND_F16 ? DT_F16 : DT_S8)); }
inline int kind_tm(int kind) { return kind == KIND_TF32 ? TM_F32 : (kind == KIND_BF16 ? TM_BF16 : (kind == KIND_F16 ? TM_F16 : TM_U8)); }
inline int kind_of_prec(int prec) { return prec == ONE_PREC_BF16 ? KIND_BF16 : (prec == ONE_PREC_F16 ? KIND_F16 : KIND_TF32); }
inline bool valid_prec(int prec) { return prec == ONE_PREC_TF32 || prec == ONE_PREC_BF16 || prec == ONE_PREC_F16; }
inline int kind_out16(int kind) { return kind == KIND_F16 ? OUT_F16 : OUT_BF16; }   // the kind's own 16-bit output mode
inline const char *kind_name(int kind) { return kind == KIND_I8 ? "s8" : (kind == KIND_BF16 ? "bf16" : (kind == KIND_F16 ? "f16" : "tf32")); }
inline int slab_for_bytes(long long row_bytes) { return row_bytes >= 128 ? 128 : (row_bytes >= 64 ? 64 : 32); }

// Split-K.  A launch with fewer output tiles than SMs leaves SMs idle, and narrowing the tile to get
// more of them wastes the tensor pipe (a 128 x 64 tf32 instruction takes as long as a 128 x 128 one).
// Instead the K blocks are cut into ranges: work unit (tile, range) writes raw fp32 partial sums into
// its own plane of a scratch buffer and a short second kernel adds the planes in a fixed order and
// applies the epilogue.  Chosen when at most half the SMs would get a tile; every range keeps at least
// 4 K blocks.  Returns the number of ranges (1: no split) and sets *kb_per_split.
int choose_split(const one_ctx *ctx, long long M, int N, int bn, int num_kb, int *kb_per_split)
{
    *kb_per_split = num_kb;
    if (!ctx->allow_split || t_split_k == 1 || num_kb < 2) return 1;
    const long long tiles = ((M + 127) / 128) * ((N + bn - 1) / bn);
    const int sms = 148;
    int want;
    if (t_split_k > 1) want = t_split_k;
    else {
        if (tiles * 2 > sms) return 1;
        want = (int)(sms / tiles);
        if (want > num_kb / 4) want = num_kb / 4;
        if (want > 16) want = 16;
    }
    if (want > num_kb) want = num_kb;
    if (want < 2) return 1;
    const int per = (num_kb + want - 1) / want;
    *kb_per_split = per;
    return (num_kb + per - 1) / per;   // every range holds at least one K block
}

// Launch `p` (epilogue fields filled in for the final output) as a split-K contraction.  Returns
// ONE_OK, an error, or 1 when the scratch for the partial sums does not fit (the caller then launches
// unsplit).
int run_split(one_ctx *ctx, int kind, int bn, const CUtensorMap &tmA, const CUtensorMap &tmB, IgemmParams p, int splits,
              int kb_per_split, cudaStream_t stream)
{
    const int Np = round_up(p.N, 32);
    const size_t plane = (size_t)p.M * Np;
    const size_t save = ctx->ws_off;
    float *partial = reinterpret_cast<float *>(ws_alloc(ctx, plane * splits * 4));
    if (!partial) {
        ctx->ws_off = save;
        return 1;
    }
    SplitKReduceParams r;
    memset(&r, 0, sizeof(r));
    r.partial = partial; r.plane_stride = (long long)plane; r.split_k = splits; r.M = p.M; r.N = p.N; r.partial_ld = Np;
    r.out = p.out; r.ldo = p.ldo; r.out_mode = p.out_mode;
    r.bias = p.bias_mode == BIAS_F32 ? reinterpret_cast<const float *>(p.bias) : nullptr;
    r.act = p.act; r.act_p0 = p.act_p0; r.act_p1 = p.act_p1; r.lut = p.lut;
    r.residual = p.residual; r.res_relu = p.res_relu; r.round_tf32 = p.round_tf32; r.status = p.status;
    // the contraction itself: raw sums, no epilogue, one plane per K range (columns padded to the store box)
    p.out = partial; p.ldo = Np; p.N = Np; p.out_mode = OUT_F32; p.bias_mode = BIAS_NONE; p.bias = nullptr;
    p.act = 0; p.lut = nullptr; p.lut_smem = 0; p.residual = nullptr; p.res_relu = 0; p.round_tf32 = 0;
    p.out_q = nullptr; p.split_k = splits; p.kb_per_split = kb_per_split; p.out_batch_stride = (long long)plane;
    p.tma_store = 1;
    CUtensorMap tmC;
    int rc = make_tmap_tiled(&tmC, TM_F32, partial, (uint64_t)Np, (uint64_t)p.M, (uint64_t)splits, (uint64_t)Np * 4, (uint64_t)plane * 4, 32, 32, 128);
    if (rc != ONE_OK) return rc;
    cudaError_t ce = launch_igemm(kind, bn, false, 1, tmA, tmB, &tmC, nullptr, p, stream);
    if (ce != cudaSuccess) return cuda_fail(ce, "igemm launch (split-K)");
    if ((ce = launch_splitk_reduce(r, stream)) != cudaSuccess) return cuda_fail(ce, "split-K reduce launch");
    return ONE_OK;
}

// Whether the final output of `p` can be produced by the split-K reduce kernel (float path, 16-byte rows).
bool split_eligible(int kind, const IgemmParams &p)
{
    if (kind == KIND_I8 || p.batched || p.out_q || !p.out || (p.out_mode != OUT_F32 && !out_is_16(p.out_mode))) return false;
    if ((p.N & 3) || (p.ldo & 3)) return false;
    return ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.residual) | reinterpret_cast<uintptr_t>(p.bias)) & 15) == 0;
}

// ---------------------------------------------------------------- descriptor parsing
int parse_conv(BUFFER_INFO_S *params, ConvGeom *g, ConvEpi *e, const CONV_CONFIG_S **cfg_out)
{
    if (!params || !params[0].addr || !params[1].addr || !params[2].addr)
        return fail(ONE_ERR_BAD_ARG, "Conv: params[0..2] must point to the config, x and W descriptors");
    const CONV_CONFIG_S *cfg = reinterpret_cast<const CONV_CONFIG_S *>(params[0].addr);
    const OPERAND_S *x = reinterpret_cast<const OPERAND_S *>(params[1].addr);
    const OPERAND_S *w = reinterpret_cast<const OPERAND_S *>(params[2].addr);
    const int yi = cfg->has_bias ? 4 : 3;   // output descriptor slot (host/op.h:127-133)
    if (!params[yi].addr) return fail(ONE_ERR_BAD_ARG, "Conv: params[%d] (output descriptor) is null", yi);
    const OPERAND_S *y = reinterpret_cast<const OPERAND_S *>(params[yi].addr);
    g->depthwise = cfg->group != 1;
    if (g->depthwise) {
        // the reference treats every group != 1 as depthwise (conv.c:29-41)
        if (cfg->group != x->shapes[1] || w->shapes[0] != x->shapes[1] || w->shapes[1] != 1)
            return fail(ONE_ERR_UNSUPPORTED, "Conv: group %lld with C %d, OC %d: only depthwise (group == C == OC) is supported",
                        (long long)cfg->group, x->shapes[1], w->shapes[0]);
    }
    g->N = x->shapes[0]; g->C = x->shapes[1]; g->H = x->shapes[2]; g->W = x->shapes[3];
    g->OC = w->shapes[0]; g->KH = w->shapes[2]; g->KW = w->shapes[3];
    g->sw = (int)cfg->strides[0]; g->sh = (int)cfg->strides[1];
    g->pt = (int)cfg->pads[0]; g->pl = (int)cfg->pads[1]; g->pb = (int)cfg->pads[2]; g->pr = (int)cfg->pads[3];
    if (g->N <= 0 || g->C <= 0 || g->H <= 0 || g->W <= 0 || g->OC <= 0 || g->KH <= 0 || g->KW <= 0)
        return fail(ONE_ERR_BAD_SHAPE, "Conv: non-positive dimension");
    if (!g->depthwise && w->shapes[1] != g->C) return fail(ONE_ERR_BAD_SHAPE, "Conv: weight C %d != input C %d", w->shapes[1], g->C);
    if (g->sw <= 0 || g->sh <= 0 || g->pt < 0 || g->pl < 0 || g->pb < 0 || g->pr < 0)
        return fail(ONE_ERR_BAD_SHAPE, "Conv: bad stride / pad");
    if ((int64_t)cfg->kernel_shape[0] != g->KH || (int64_t)cfg->kernel_shape[1] != g->KW)
        return fail(ONE_ERR_BAD_SHAPE, "Conv: kernel_shape %lldx%lld != weight %dx%d", (long long)cfg->kernel_shape[0],
                    (long long)cfg->kernel_shape[1], g->KH, g->KW);
    e->int8 = (cfg->ifmap_quant2 == TYPE_INT8);
    if (e->int8) {
        if (g->pl != g->pt || g->pb != g->pt || g->pr != g->pt)
            return fail(ONE_ERR_UNSUPPORTED, "Conv int8: the reference pads every side by pads[0]; unequal pads are rejected");
        if (g->OC > ONE_WEIGHT_AUX_LEN) return fail(ONE_ERR_BAD_SHAPE, "Conv int8: OC %d > %d (weight_aux)", g->OC, ONE_WEIGHT_AUX_LEN);
        // a negative scale is legal in the reference (its percent calibrator can produce one): x / s is
        // quantised and acc * s restores the sign; only 0 and non-finite values have no meaning
        if (cfg->input_scale == 0.f || !isfinite(cfg->input_scale)) return fail(ONE_ERR_BAD_ARG, "Conv int8: input_scale must be finite and non-zero");
    }
    if (g->H + g->pt + g->pb < g->KH || g->W + g->pl + g->pr < g->KW) return fail(ONE_ERR_BAD_SHAPE, "Conv: kernel larger than padded input");
    g->OH = (g->H + g->pt + g->pb - g->KH) / g->sh + 1;   // host/ops/conv.h:44-47
    g->OW = (g->W + g->pl + g->pr - g->KW) / g->sw + 1;
    if (y->shapes[1] != g->OC || y->shapes[2] != g->OH || y->shapes[3] != g->OW)
        return fail(ONE_ERR_BAD_SHAPE, "Conv: output descriptor [%d,%d,%d] != computed [%d,%d,%d]", y->shapes[1], y->shapes[2],
                    y->shapes[3], g->OC, g->OH, g->OW);
    if ((long long)g->N * g->OH * g->OW > 0x7fffffffLL) return fail(ONE_ERR_BAD_SHAPE, "Conv: too many output pixels");
    e->has_bias = cfg->has_bias ? 1 : 0;
    e->act = e->has_bias ? (int)cfg->act_type : 0;   // bias-less conv: no activation (conv.c:18-27)
    e->p0 = e->p1 = 0.f;
    if (e->act == CLIP) { e->p0 = cfg->clip_min; e->p1 = cfg->clip_max; }
    else if (e->act == LEAKYRELU) e->p0 = cfg->leaky_relu_alpha;
    else if (e->act == HARDSILU) { e->p0 = cfg->hard_sigmoid_alpha; e->p1 = cfg->hard_sigmoid_beta; }
    e->in_scale = cfg->input_scale;
    *cfg_out = cfg;
    return ONE_OK;
}

// Geometry of the space-to-depth rewrite; false when it does not apply.
bool s2d_plan(const ConvGeom &g, ConvPlan *p)
{
    p->eh = g.pt & 1; p->ew = g.pl & 1;
    const int Ph = (g.pt + p->eh) / 2, Pw = (g.pl + p->ew) / 2;
    // four columns per position when they still fit one 128-byte row and the filter is wide enough
    p->bw = (8 * g.C * p->es <= 128 && g.C <= 4 && g.KW + p->ew > 2 && Pw >= 1) ? 4 : 2;
    p->dil_w = p->bw / 2;
    p->KH2 = (g.KH - 1 + p->eh) / 2 + 1;
    p->KW2 = (g.KW + p->ew + p->bw - 1) / p->bw;
    const int ext_w = (p->KW2 - 1) * p->dil_w + 1;   // positions spanned along w
    const int off = p->bw / 2 - 1;   // positions the overlapping layout starts left of the image
    p->Hs = (g.H + 1) / 2; p->Ws = (g.W + 1) / 2 + off;
    {   // channel slots per position: the row is 32, 64 or 128 bytes wide (one swizzle span)
        const int cb = 2 * p->bw * g.C * p->es;
        p->Cp = (cb <= 32 ? 32 : (cb <= 64 ? 64 : 128)) / p->es;
    }
    p->pt2 = Ph; p->pl2 = Pw - off;
    // overlapping layout: exactly the positions some output needs (the packer zero-fills past the image)
    if (p->bw == 4) p->Ws = g.OW - p->pl2 + ext_w - 1;
    p->pb2 = g.OH - p->Hs - Ph + p->KH2 - 1;
    p->pr2 = g.OW - p->Ws - p->pl2 + ext_w - 1;
    return p->pb2 >= 0 && p->pr2 >= 0 && p->pl2 >= 0 && p->pb2 < p->KH2 && p->pr2 < ext_w && Ph <= 128 && Pw <= 128;
}

// Path selection.  x_is_nchw_f32: the activation arrives in the reference layout and has to be
// re-laid anyway, so the explicit-im2col fallback can read it directly.
void plan_conv(const ConvGeom &g, int kind, ConvPlan *p, bool x_nchw_f32)
{
    p->kind = kind; p->es = kind_es(kind); p->adt = kind_dt(kind);
    const int K = g.C * g.KH * g.KW;
    const long long cbytes = (long long)g.C * p->es;
    const bool one_by_one = g.KH == 1 && g.KW == 1 && g.sw == 1 && g.sh == 1 && !g.pt && !g.pl && !g.pb && !g.pr;
    const bool corners_ok = g.pl <= 128 && g.pt <= 128 && (g.pr - (g.KW - 1)) >= -128 && (g.pb - (g.KH - 1)) >= -128 &&
                            g.pr - (g.KW - 1) <= 127 && g.pb - (g.KH - 1) <= 127 && g.sw <= 8 && g.sh <= 8 && g.KW <= 65535;
    if (one_by_one && cbytes % 16 == 0) {
        p->path = PATH_TILED;
        p->w_pitch = g.C;
        p->slab_bytes = slab_for_bytes(cbytes);
        p->num_kb = (int)((cbytes + p->slab_bytes - 1) / p->slab_bytes);
        p->c_slabs = p->num_kb;
    } else if (cbytes % 32 == 0 && corners_ok) {
        p->path = PATH_IM2COL;
        p->w_pitch = K;
        p->slab_bytes = (cbytes % 128 == 0) ? 128 : (cbytes % 64 == 0 ? 64 : 32);
        p->c_slabs = (int)(cbytes / p->slab_bytes);
        p->num_kb = g.KH * g.KW * p->c_slabs;
    } else if (x_nchw_f32 && g.sw == 2 && g.sh == 2 && 4 * cbytes <= 128 && s2d_plan(g, p)) {
        // a few-channel stride-2 conv on the network input (ResNet's 7x7 stem): ih = 2*oh + kh - pt is
        // rewritten as 2*(oh + a - P) + b with kh + e = 2a + b, e = pt mod 2, P = (pt + e)/2, which is a
        // stride-1 conv with a (KH+e+1)/2-tap filter over the space-to-depth image whose channel index
        // is (b_h, b_w, c).  No im2col matrix is materialised: the tensor-map path reads that image.
        p->path = PATH_S2D;
        p->w_pitch = p->KH2 * p->KW2 * p->Cp;
        const long long cb = (long long)p->Cp * p->es;
        p->slab_bytes = (cb % 128 == 0) ? 128 : (cb % 64 == 0 ? 64 : 32);
        p->c_slabs = (int)(cb / p->slab_bytes);
        p->num_kb = p->KH2 * p->KW2 * p->c_slabs;
    } else if (x_nchw_f32 && kind != KIND_I8 && g.KH == g.sh && g.KW == g.sw && !g.pt && !g.pl && !g.pb && !g.pr &&
               g.H % g.KH == 0 && g.W % g.KW == 0 && g.KW % 4 == 0) {
        // non-overlapping patches on the network input (a ViT patch embedding): the im2col matrix is a
        // re-ordering of the image with K running (c, kh, kw), the order of the weight tensor itself
        p->path = PATH_PATCH;
        p->w_pitch = round_up(K, 32 / p->es);
        p->slab_bytes = slab_for_bytes((long long)p->w_pitch * p->es);
        p->num_kb = (p->w_pitch * p->es + p->slab_bytes - 1) / p->slab_bytes;
        p->c_slabs = p->num_kb;
    } else {
        p->path = PATH_EXPLICIT;
        p->w_pitch = round_up(K, 32 / p->es);
        p->slab_bytes = slab_for_bytes((long long)p->w_pitch * p->es);
        p->num_kb = (p->w_pitch * p->es + p->slab_bytes - 1) / p->slab_bytes;
        p->c_slabs = p->num_kb;
    }
    p->slab_elems = p->slab_bytes / p->es;
    const int code = pick_bn(g.OC, (long long)g.N * g.OH * g.OW);
    p->bn = tile_bn(code);
    p->cta2 = tile_cta2(code) ? 1 : 0;
    p->mh = tile_mh(code);
    p->nw = tile_nw(code);
}

// Width pairing.  A 128 x 64 tensor-core instruction takes as long as a 128 x 128 one, so a convolution
// with 64 (or fewer) output channels runs the tensor pipe at half rate.  For a stride-1 multi-tap filter
// two horizontally adjacent output pixels are computed as ONE row of the contraction instead: the pair
// (ow = 2q, 2q + 1) reads the input window of KW + 1 columns starting at 2q - pad_l, output channel block
// j (pixel 2q + j) uses taps kw' - j of it and zero elsewhere.  That is a convolution with a KH x (KW + 1)
// filter, stride 2 along w, one more column of right padding and 2 * OC output channels, whose NHWC output
// [N][OH][OW / 2][2 * OC] is byte for byte the original [N][OH][OW][OC]: M halves, N doubles, K grows by
// (KW + 1) / KW, i.e. the tensor pipe and the L2 -> SM activation stream both do 2/3 of the work for a 3 x 3
// filter.  The extra products are exact zeros (x * 0.0f), so each output sums the same terms; only their
// grouping inside the tensor core changes.  Applies to the device-resident NHWC float path; bias,
// activation, residual and rounding are per element and carry over with the bias stored twice.
bool pair_geometry(const ConvGeom &g, const ConvEpi &e, int es, ConvGeom *gp)
{
    if (!t_pairing || e.int8 || g.depthwise) return false;
    if (g.OC > 64 || g.OC % 32 || g.sw != 1 || g.sh != 1 || g.KW < 2 || (g.OW & 1)) return false;
    if (((long long)g.C * es) % 32) return false;          // the tensor-map (im2col) path must apply
    *gp = g;
    gp->OC = 2 * g.OC;
    gp->KW = g.KW + 1;
    gp->sw = 2;
    gp->pr = g.pr + 1;
    gp->OW = g.OW / 2;
    return true;
}

// Host side of the pairing: OIHW weights [OC][C][KH][KW] -> [2 * OC][C][KH][KW + 1].
void pair_weights(const float *w, const ConvGeom &g, std::vector<float> *out)
{
    const int KW2 = g.KW + 1;
    out->assign((size_t)2 * g.OC * g.C * g.KH * KW2, 0.f);
    for (int j = 0; j < 2; ++j)
        for (int oc = 0; oc < g.OC; ++oc)
            for (int c = 0; c < g.C; ++c)
                for (int kh = 0; kh < g.KH; ++kh)
                    for (int kw = 0; kw < g.KW; ++kw)
                        (*out)[((((size_t)(j * g.OC + oc) * g.C + c) * g.KH + kh) * KW2) + kw + j] =
                            w[(((size_t)oc * g.C + c) * g.KH + kh) * g.KW + kw];
}

// Re-order the weights for the plan's path.
cudaError_t pack_weights_for(const ConvGeom &g, const ConvPlan &pl, const void *w_src, void *w_dst, int src_is_s8, cudaStream_t st)
{
    if (pl.path == PATH_PATCH)   // K order (c, kh, kw): the weight rows as they are, padded to the pitch
        return pack_rows(reinterpret_cast<const float *>(w_src), w_dst, g.OC, g.C * g.KH * g.KW, pl.w_pitch, pl.adt, st);
    if (pl.path == PATH_S2D)
        return pack_conv_weight_s2d(w_src, w_dst, g.OC, g.C, g.KH, g.KW, pl.KH2, pl.KW2, pl.eh, pl.ew, pl.Cp, pl.bw, pl.adt, src_is_s8, st);
    return pack_conv_weight(w_src, w_dst, g.OC, g.C, g.KH, g.KW, pl.w_pitch, pl.adt, src_is_s8, st);
}

struct ConvIO {
    const void *x;        // NHWC in plan.adt, or NCHW f32 when x_nchw_f32
    int x_nchw_f32;
    const void *w;        // packed [OC][w_pitch] in plan.adt
    const void *bias;     // f32[OC] or s32[OC] (int8), device
    const float *coeff;   // int8 de-quantisation coefficients, device
    const float *lut;     // SiLU table, device
    void *y;              // NHWC
    int out_mode;         // OUT_F32 / OUT_BF16 / OUT_RAW32
    const void *residual;
    int res_relu;
    int round_tf32;
    int8_t *out_q;
    float q_inv_scale;
    float x_inv_scale;    // int8 + x_nchw_f32 explicit path: quantise while packing
};

// Store map for the epilogue's TMA path; *use is set to 1 when the output qualifies (no int8 copy, N a
// multiple of 32, 16-byte aligned rows), to 2 when the int8 copy is the only output.
int make_store_map(int kind, CUtensorMap *m, CUtensorMap *mres, int *use, void *out, int out_mode, long long M, int N, long long ldo,
                   int batch, long long out_bstride, const void *residual, const void *out_q)
{
    *use = 0;
    if (!out && out_q && !residual && (N % 32) == 0 && (ldo % 16) == 0 && (out_bstride % 16) == 0 &&
        (reinterpret_cast<uintptr_t>(out_q) & 15) == 0) {
        // int8-only output (the quantised activation of an int8 chain): 32 x 32-byte patches, no swizzle
        int rc = make_tmap_tiled(m, TM_U8, out_q, (uint64_t)N, (uint64_t)M, (uint64_t)batch, (uint64_t)ldo, (uint64_t)out_bstride,
                                 32, 32, 0);
        if (rc != ONE_OK) return rc;
        *use = 2;
        return ONE_OK;
    }
    if (!out || out_q || (out_mode != OUT_F32 && !out_is_16(out_mode)) || (N % 32) != 0) return ONE_OK;
    const int es = out_is_16(out_mode) ? 2 : 4;
    if ((ldo * es) % 16 || (out_bstride * es) % 16 || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (reinterpret_cast<uintptr_t>(residual) & 15))
        return ONE_OK;
    // A box is 32 rows of 32 columns; the 16-bit kinds write a 16-bit output as 64-column boxes (128-byte rows,
    // computed as two 32-column halves; the store clips a second half that lies beyond N).
    const int tm = out_mode == OUT_BF16 ? TM_BF16 : (out_mode == OUT_F16 ? TM_F16 : TM_F32);
    const uint32_t box_cols = (out_is_16(out_mode) && kind_is_16(kind)) ? 64 : 32;
    const uint32_t sw = box_cols * es;   // 128, or 64 for a 32-column 16-bit box
    if ((uint32_t)N < box_cols) return ONE_OK;
    int rc = make_tmap_tiled(m, tm, out, (uint64_t)N, (uint64_t)M, (uint64_t)batch, (uint64_t)ldo * es,
                             (uint64_t)out_bstride * es, box_cols, 32, sw);
    if (rc == ONE_OK && residual)
        rc = make_tmap_tiled(mres, tm, residual, (uint64_t)N, (uint64_t)M, (uint64_t)batch, (uint64_t)ldo * es,
                             (uint64_t)out_bstride * es, box_cols, 32, sw);
    if (rc != ONE_OK) return rc;
    *use = 1;
    return ONE_OK;
}

// The TMA-store epilogue reads the bias and the int8 coefficients 16 bytes at a time; the reference
// accepts any float-aligned bias, so a caller's pointer that is only 4- or 8-byte aligned goes down the
// transposing path, which loads such constants one by one.
inline bool vec_constants_ok(const IgemmParams &p)
{
    return ((reinterpret_cast<uintptr_t>(p.bias) | reinterpret_cast<uintptr_t>(p.coeff)) & 15) == 0;
}

// Enqueue one convolution.  `amap` (optional) caches the A tensor map between calls.
int run_conv(one_ctx *ctx, const ConvGeom &g, const ConvEpi &e, const ConvPlan &pl, const ConvIO &io,
             const CUtensorMap *tmB_cached, cudaStream_t stream)
{
    const long long M = (long long)g.N * g.OH * g.OW;
    CUtensorMap tmA, tmB;
    int rc;
    if (pl.path == PATH_EXPLICIT) {
        void *col = ws_alloc(ctx, (size_t)M * pl.w_pitch * pl.es);
        if (!col) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the %lld x %d im2col matrix", M, pl.w_pitch);
        cudaError_t ce = im2col_pack(io.x, col, g.N, g.C, g.H, g.W, g.KH, g.KW, g.OH, g.OW, g.sw, g.sh, g.pt, g.pl,
                                     pl.w_pitch, io.x_nchw_f32 ? 0 : 1, io.x_nchw_f32 ? DT_F32 : pl.adt, pl.adt,
                                     io.x_inv_scale, stream);
        if (ce != cudaSuccess) return cuda_fail(ce, "im2col_pack");
        rc = make_tmap_tiled(&tmA, kind_tm(pl.kind), col, pl.w_pitch, M, 0, (uint64_t)pl.w_pitch * pl.es, 0,
                             pl.slab_elems, 128, pl.slab_bytes);
    } else if (pl.path == PATH_PATCH) {
        void *col = ws_alloc(ctx, (size_t)M * pl.w_pitch * pl.es);
        if (!col) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the %lld x %d patch matrix", M, pl.w_pitch);
        cudaError_t ce = patch_pack(reinterpret_cast<const float *>(io.x), col, g.N, g.C, g.H, g.W, g.KH, g.KW, pl.w_pitch, pl.adt, stream);
        if (ce != cudaSuccess) return cuda_fail(ce, "patch_pack");
        rc = make_tmap_tiled(&tmA, kind_tm(pl.kind), col, pl.w_pitch, M, 0, (uint64_t)pl.w_pitch * pl.es, 0,
                             pl.slab_elems, 128, pl.slab_bytes);
    } else if (pl.path == PATH_S2D) {
        void *img = ws_alloc(ctx, (size_t)g.N * pl.Hs * pl.Ws * pl.Cp * pl.es);
        if (!img) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the space-to-depth image");
        cudaError_t ce = s2d_pack(reinterpret_cast<const float *>(io.x), img, g.N, g.C, g.H, g.W, pl.Hs, pl.Ws, pl.Cp, pl.bw, pl.adt,
                                  io.x_inv_scale, stream);
        if (ce != cudaSuccess) return cuda_fail(ce, "s2d_pack");
        rc = make_tmap_im2col(&tmA, kind_tm(pl.kind), img, pl.Cp, pl.Ws, pl.Hs, g.N, pl.pl2, pl.pt2, pl.pr2, pl.pb2,
                              (pl.KW2 - 1) * pl.dil_w + 1 /* positions spanned along w */, pl.KH2, 1, 1, pl.slab_elems, 128,
                              pl.slab_bytes);
    } else if (pl.path == PATH_TILED) {
        rc = make_tmap_tiled(&tmA, kind_tm(pl.kind), io.x, g.C, M, 0, (uint64_t)g.C * pl.es, 0, pl.slab_elems, 128,
                             pl.slab_bytes);
    } else {
        rc = make_tmap_im2col(&tmA, kind_tm(pl.kind), io.x, g.C, g.W, g.H, g.N, g.pl, g.pt, g.pr, g.pb, g.KW, g.KH,
                              g.sw, g.sh, pl.slab_elems, 128, pl.slab_bytes);
    }
    if (rc != ONE_OK) return rc;
    if (tmB_cached) tmB = *tmB_cached;
    else {
        rc = make_tmap_tiled(&tmB, kind_tm(pl.kind), io.w, pl.w_pitch, g.OC, 0, (uint64_t)pl.w_pitch * pl.es, 0,
                             pl.slab_elems, pl.cta2 ? pl.bn / 2 : pl.bn, pl.slab_bytes);
        if (rc != ONE_OK) return rc;
    }
    IgemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = (int)M; p.N = g.OC; p.num_kb = pl.num_kb; p.slab_bytes = pl.slab_bytes; p.slab_elems = pl.slab_elems;
    p.a_im2col = pl.path == PATH_IM2COL || pl.path == PATH_S2D;
    p.OW = g.OW; p.OH = g.OH; p.stride_w = g.sw; p.stride_h = g.sh; p.pad_l = g.pl; p.pad_t = g.pt;
    p.KW = g.KW; p.KH = g.KH; p.c_slabs = pl.c_slabs;
    p.dil_w = 1;
    if (pl.path == PATH_S2D) {
        p.stride_w = p.stride_h = 1; p.pad_l = pl.pl2; p.pad_t = pl.pt2; p.KW = pl.KW2; p.KH = pl.KH2;
        p.dil_w = pl.dil_w;
    }
    p.out = io.y; p.ldo = g.OC; p.out_mode = io.out_mode;
    if (pl.kind == KIND_I8) {
        p.bias_mode = BIAS_S32_DEQUANT; p.bias = e.has_bias ? io.bias : nullptr;
        p.coeff = io.coeff; p.in_scale = e.in_scale;
    } else {
        p.bias_mode = e.has_bias ? BIAS_F32 : BIAS_NONE; p.bias = io.bias;
    }
    p.act = e.act; p.act_p0 = e.p0; p.act_p1 = e.p1; p.lut = io.lut;
    p.residual = io.residual; p.res_relu = io.res_relu; p.round_tf32 = io.round_tf32;
    p.lut_smem = p.act == SILU && p.lut && !p.residual && (reinterpret_cast<uintptr_t>(p.lut) & 15) == 0;
    p.out_q = io.out_q; p.q_inv_scale = io.q_inv_scale;
    p.status = ctx->status_dev;
    if (!pl.cta2 && pl.mh == 1 && pl.nw == 8 && split_eligible(pl.kind, p)) {
        int per = 0;
        const int splits = choose_split(ctx, M, g.OC, pl.bn, pl.num_kb, &per);
        if (splits > 1 && (rc = run_split(ctx, pl.kind, pl.bn, tmA, tmB, p, splits, per, stream)) != 1) {
            t_last_split = splits;
            return rc;
        }
    }
    t_last_split = 1;
    CUtensorMap tmC, tmR, tmI;
    // Residual added by the tensor core (bit 3 of the epilogue mode): a 16-bit residual of the operands' own
    // format, no activation between the convolution and the Add, plain 256-wide tiles on full 128-byte slabs
    // (on narrower tiles the extra operand stages cost more than the epilogue saves: measured).  The
    // residual tensor becomes an operand (64-column x 128-row boxes) multiplied by an identity tile; what is
    // left for the epilogue is bias (+ the ReLU that followed the Add).  (a + r) + b instead of (a + b) + r: the
    // same terms in fp32, rounding of the last bit aside.
    const bool res_mma = p.residual && (get_epilogue_mode() & 8) && kind_is_16(pl.kind) && p.out_mode == kind_out16(pl.kind) && p.act == 0 &&
                         !pl.cta2 && pl.mh == 1 && pl.nw == 8 && pl.bn == 256 && pl.slab_bytes == 128 && g.OC % 64 == 0 && !p.out_q && ctx->ident16[0] &&
                         (p.ldo * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0;
    const void *residual = p.residual;
    if (res_mma) {
        p.residual = nullptr;
        p.act = p.res_relu ? RELU : 0;
        p.res_relu = 0;
    }
    if ((rc = make_store_map(pl.kind, &tmC, &tmR, &p.tma_store, p.out, p.out_mode, M, g.OC, p.ldo, 0, 0, p.residual, p.out_q)) != ONE_OK) return rc;
    if (!vec_constants_ok(p)) p.tma_store = 0;
    if (res_mma) {
        const int f = pl.kind == KIND_F16 ? 1 : 0;
        if ((rc = make_tmap_tiled(&tmR, kind_tm(pl.kind), residual, (uint64_t)g.OC, (uint64_t)M, 0, (uint64_t)p.ldo * 2, 0, 64, 128, 128)) != ONE_OK ||
            (rc = make_tmap_tiled(&tmI, kind_tm(pl.kind), ctx->ident16[f], 64, 64, 0, 128, 0, 64, 64, 128)) != ONE_OK)
            return rc;
        p.res_mma = 1;
    }
    cudaError_t ce = launch_igemm(pl.kind, pl.bn, pl.cta2 != 0, pl.mh, tmA, tmB, p.tma_store ? &tmC : nullptr,
                                  (res_mma || (p.tma_store && p.residual)) ? &tmR : nullptr, p, stream, res_mma ? &tmI : nullptr, pl.nw);
    if (ce != cudaSuccess) return cuda_fail(ce, "igemm launch");
    return ONE_OK;
}

// Depthwise convolution straight on the reference layout (no scratch): CUDA cores, HBM bound.
// int8 (e.int8): w is int8, bias int32, aux = weight_aux on the device.
int run_depthwise(const ConvGeom &g, const ConvEpi &e, const float *x, const void *w, const void *bias, const float *aux,
                  const float *lut, float *y, cudaStream_t stream)
{
    cudaError_t ce;
    if (e.int8)
        ce = dwconv_s8_nchw(x, reinterpret_cast<const int8_t *>(w), e.has_bias ? reinterpret_cast<const int *>(bias) : nullptr, aux,
                            y, g.N, g.C, g.H, g.W, g.OH, g.OW, g.KH, g.KW, g.sw, g.sh, g.pt, e.in_scale, e.act, e.p0, e.p1, lut,
                            stream);
    else
        ce = dwconv_nchw(x, reinterpret_cast<const float *>(w), e.has_bias ? reinterpret_cast<const float *>(bias) : nullptr, y,
                         g.N, g.C, g.H, g.W, g.OH, g.OW, g.KH, g.KW, g.sw, g.sh, g.pt, g.pl, e.act, e.p0, e.p1, lut, stream);
    return ce == cudaSuccess ? ONE_OK : cuda_fail(ce, "dwconv launch");
}

// weight_aux of an int8 depthwise conv, copied into the call's scratch; null for fp32.
int depthwise_aux(one_ctx *ctx, const ConvGeom &g, const ConvEpi &e, const CONV_CONFIG_S *cfg, const float **aux, cudaStream_t st)
{
    *aux = nullptr;
    if (!e.int8) return ONE_OK;
    float *ad = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)g.OC * 4));
    if (!ad) return fail(ONE_ERR_NOMEM, "Conv: workspace too small (weight_aux)");
    cudaError_t ce = cudaMemcpyAsync(ad, cfg->weight_aux, (size_t)g.OC * 4, cudaMemcpyHostToDevice, st);
    if (ce != cudaSuccess) return cuda_fail(ce, "weight_aux upload");
    *aux = ad;
    return ONE_OK;
}

// Epilogue extras of a fused linear layer: table activation, residual add.
struct GemmEpi {
    int act = NOT_ACT;
    const float *lut = nullptr;
    const void *residual = nullptr;   // [M][ldo], same type as the output
};

// Plain GEMM D[M,N] = A[M,K] * B[N,K]^T (+bias, +activation, +residual), optionally batched.
int run_gemm(one_ctx *ctx, int kind, const void *A, int a_pitch, const void *B, int b_pitch, long long M, int N,
             int K, int batch, long long a_bstride, long long b_bstride, void *out, long long ldo,
             long long out_bstride, int out_mode, const float *bias, const CUtensorMap *tmB_cached, int bn,
             cudaStream_t stream, const GemmEpi *epi = nullptr)
{
    if (M > 0x7fffffffLL) return fail(ONE_ERR_BAD_SHAPE, "GEMM: M too large");
    const bool cta2 = tile_cta2(bn) && batch == 0;   // `bn` arrives as a tile code; a batched product stays single-CTA
    const int mh = tile_mh(bn), nw = batch == 0 ? tile_nw(bn) : 8;
    bn = tile_bn(bn);
    const int es = kind_es(kind);
    const int slab_bytes = slab_for_bytes((long long)K * es);
    const int slab_elems = slab_bytes / es;
    CUtensorMap tmA, tmB;
    int rc = make_tmap_tiled(&tmA, kind_tm(kind), A, K, M, batch, (uint64_t)a_pitch * es, (uint64_t)a_bstride * es,
                             slab_elems, 128, slab_bytes);
    if (rc != ONE_OK) return rc;
    if (tmB_cached) tmB = *tmB_cached;
    else {
        rc = make_tmap_tiled(&tmB, kind_tm(kind), B, K, N, batch, (uint64_t)b_pitch * es, (uint64_t)b_bstride * es,
                             slab_elems, cta2 ? bn / 2 : bn, slab_bytes);
        if (rc != ONE_OK) return rc;
    }
    IgemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = (int)M; p.N = N; p.num_kb = (int)(((long long)K * es + slab_bytes - 1) / slab_bytes);
    p.slab_bytes = slab_bytes; p.slab_elems = slab_elems;
    p.batched = batch > 0; p.batch = batch; p.out_batch_stride = out_bstride;
    p.out = out; p.ldo = ldo; p.out_mode = out_mode;
    p.bias_mode = bias ? BIAS_F32 : BIAS_NONE; p.bias = bias;
    if (epi) { p.act = epi->act; p.lut = epi->lut; p.residual = epi->residual; }
    p.lut_smem = p.act == SILU && p.lut && !p.residual && (reinterpret_cast<uintptr_t>(p.lut) & 15) == 0;
    p.status = ctx->status_dev;
    if (!cta2 && mh == 1 && nw == 8 && split_eligible(kind, p)) {
        int per = 0;
        const int splits = choose_split(ctx, M, N, bn, p.num_kb, &per);
        if (splits > 1 && (rc = run_split(ctx, kind, bn, tmA, tmB, p, splits, per, stream)) != 1) {
            t_last_split = splits;
            return rc;
        }
    }
    t_last_split = 1;
    CUtensorMap tmC, tmR;
    if ((rc = make_store_map(kind, &tmC, &tmR, &p.tma_store, out, out_mode, M, N, ldo, batch, out_bstride, p.residual, nullptr)) != ONE_OK) return rc;
    if (!vec_constants_ok(p)) p.tma_store = 0;
    cudaError_t ce = launch_igemm(kind, bn, cta2, mh, tmA, tmB, p.tma_store ? &tmC : nullptr, (p.tma_store && p.residual) ? &tmR : nullptr, p, stream, nullptr, nw);
    if (ce != cudaSuccess) return cuda_fail(ce, "igemm launch");
    return ONE_OK;
}

}  // namespace

// A timeout outranks a range report: after a stalled role the values are not meaningful anyway.
int one::status_fail(unsigned int st)
{
    if (st == one::ST_RANGE_F16)
        return fail(ONE_ERR_RANGE, "a value written as fp16 exceeded the format's range (65504): run this model with ONE_PREC_TF32");
    return fail(ONE_ERR_TIMEOUT, "device-side wait ran out (status word 0x%x)", st);
}

namespace {

int finish_sync(one_ctx *ctx, cudaStream_t stream)
{
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return cuda_fail(e, "stream synchronise");
    unsigned int st = 0;
    if ((e = cudaMemcpy(&st, ctx->status_dev, sizeof(st), cudaMemcpyDeviceToHost)) != cudaSuccess)
        return cuda_fail(e, "status read");
    if (st) {
        cudaMemset(ctx->status_dev, 0, sizeof(st));
        return status_fail(st);
    }
    return ONE_OK;
}

// int8 de-quantisation coefficients exactly as the reference forms them:
// weight_aux[oc] * 1 / 127.0f  (device/x86/Conv/conv.c:1052).
void dequant_coeffs(const CONV_CONFIG_S *cfg, int OC, std::vector<float> *out)
{
    out->resize(OC);
    for (int i = 0; i < OC; ++i) (*out)[i] = cfg->weight_aux[i] * 1 / 127.0f;
}

inline size_t up256(size_t v) { return (v + 255) & ~size_t(255); }

// Scratch a drop-in Conv call carves out of the workspace (reference layout in and out), counted the
// way ws_alloc hands it out, so that a call that cannot fit is refused before anything is launched.
size_t conv_eval_scratch(const ConvGeom &g, const ConvEpi &e, const ConvPlan &pl)
{
    const long long M = (long long)g.N * g.OH * g.OW;
    size_t need = 0;
    if (pl.path == PATH_EXPLICIT || pl.path == PATH_PATCH) need += up256((size_t)M * pl.w_pitch * pl.es);
    else if (pl.path == PATH_S2D) need += up256((size_t)g.N * pl.Hs * pl.Ws * pl.Cp * pl.es);
    else need += up256((size_t)g.N * g.H * g.W * g.C * pl.es);
    need += up256((size_t)g.OC * pl.w_pitch * pl.es) + up256((size_t)M * g.OC * 4);
    if (e.int8) need += 2 * up256((size_t)g.OC * 4);
    return need;
}

struct MatmulShape {
    int batch, M, K, N, b_shared;
};
int parse_matmul(BUFFER_INFO_S *params, MatmulShape *s)
{
    if (!params || !params[1].addr || !params[2].addr || !params[3].addr)
        return fail(ONE_ERR_BAD_ARG, "MatMul: params[1..3] must point to the A, B and Y descriptors");
    const OPERAND_S *a = reinterpret_cast<const OPERAND_S *>(params[1].addr);
    const OPERAND_S *b = reinterpret_cast<const OPERAND_S *>(params[2].addr);
    const OPERAND_S *y = reinterpret_cast<const OPERAND_S *>(params[3].addr);
    if (a->dim_num_of_shapes < 2 || a->dim_num_of_shapes > SHAPE_LEN || y->dim_num_of_shapes < 1 ||
        y->dim_num_of_shapes > SHAPE_LEN)
        return fail(ONE_ERR_BAD_SHAPE, "MatMul: A needs at least 2 dims");
    long long batch = 1;
    for (int i = 0; i < a->dim_num_of_shapes - 2; ++i) batch *= a->shapes[i];   // mat_mul.c:24-27
    s->M = a->shapes[a->dim_num_of_shapes - 2];
    s->K = a->shapes[a->dim_num_of_shapes - 1];
    s->N = y->shapes[y->dim_num_of_shapes - 1];
    long long b_elems = 1;
    for (int i = 0; i < SHAPE_LEN; ++i) b_elems *= b->shapes[i];
    if (batch <= 0 || batch > 0x7fffffff || s->M <= 0 || s->K <= 0 || s->N <= 0)
        return fail(ONE_ERR_BAD_SHAPE, "MatMul: non-positive dimension");
    s->batch = (int)batch;
    s->b_shared = (b_elems == (long long)s->K * s->N);   // mat_mul.c:42-46
    if (!s->b_shared && b_elems != batch * s->K * s->N)
        return fail(ONE_ERR_BAD_SHAPE, "MatMul: B has %lld elements, expected %lld or %lld", b_elems, (long long)s->K * s->N,
                    batch * s->K * s->N);
    return ONE_OK;
}

}  // namespace

// ============================================================================ drop-in evals
extern "C" int one_cuda_set_eval_precision(int prec)
{
    if (!valid_prec(prec)) return fail(ONE_ERR_BAD_ARG, "unknown precision %d", prec);
    t_eval_prec = prec;
    return ONE_OK;
}

extern "C" int one_cuda_selftest_wait_timeout(one_ctx *ctx, unsigned long long limit_clocks)
{
    if (!ctx) return fail(ONE_ERR_BAD_ARG, "null context");
    if (limit_clocks == 0 || limit_clocks > (1ull << 31)) return fail(ONE_ERR_BAD_ARG, "limit must be in (0, 2^31] clocks");
    cudaError_t ce = launch_wait_probe(ctx->status_dev, (long long)limit_clocks, ctx->stream);
    return ce == cudaSuccess ? ONE_OK : cuda_fail(ce, "wait probe launch");
}

extern "C" int one_cuda_set_tile_n(int bn)
{
    if (bn != 0 && !valid_tile(bn)) return fail(ONE_ERR_BAD_ARG, "tile must be 0, 64, 128, 192, 256, 1128 / 1192 / 1256 (pairs of CTAs), 2064 / 2128 (two 128-row halves per CTA) or 4064 / 4128 (twelve epilogue warps)");
    if (tile_cta2(bn) && !g_cta_pairs.load(std::memory_order_relaxed)) return fail(ONE_ERR_UNSUPPORTED, "pairs of CTAs are switched off (one_cuda_set_cta_pairs)");
    if (tile_mh(bn) == 2 && !g_half_tiles.load(std::memory_order_relaxed)) return fail(ONE_ERR_UNSUPPORTED, "two-half tiles are switched off (one_cuda_set_half_tiles)");
    if (tile_nw(bn) == 12 && !g_wide_epi.load(std::memory_order_relaxed)) return fail(ONE_ERR_UNSUPPORTED, "twelve-warp epilogues are switched off (one_cuda_set_wide_epilogue)");
    t_tile_n = bn;
    return ONE_OK;
}

extern "C" int one_cuda_set_split_k(int splits)
{
    if (splits < 0 || splits > 64) return fail(ONE_ERR_BAD_ARG, "split count must be 0 (library's choice), 1 (never) or 2..64");
    t_split_k = splits;
    return ONE_OK;
}

extern "C" int one_cuda_set_wide_epilogue(int on)
{
    g_wide_epi.store(on ? 1 : 0, std::memory_order_relaxed);
    return ONE_OK;
}

extern "C" int one_cuda_set_half_tiles(int on)
{
    g_half_tiles.store(on ? 1 : 0, std::memory_order_relaxed);
    return ONE_OK;
}

extern "C" int one_cuda_set_cta_pairs(int on)
{
    g_cta_pairs.store(on ? 1 : 0, std::memory_order_relaxed);
    return ONE_OK;
}

extern "C" int one_cuda_set_epilogue_mode(int bits)
{
    set_epilogue_mode(bits);
    return ONE_OK;
}

extern "C" int one_cuda_set_width_pairing(int on)
{
    t_pairing = on ? 1 : 0;
    return ONE_OK;
}

extern "C" int one_cuda_set_launch_overlap(int on)
{
    set_pdl(on);
    return ONE_OK;
}

extern "C" int one_cuda_conv_eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs)
{
    ConvGeom g; ConvEpi e; const CONV_CONFIG_S *cfg;
    int rc = parse_conv(params, &g, &e, &cfg);
    if (rc != ONE_OK) return rc;
    if (!inputs || !outputs || !inputs[0].addr || !inputs[1].addr || !outputs[0].addr || (e.has_bias && !inputs[2].addr))
        return fail(ONE_ERR_BAD_ARG, "Conv: null tensor pointer");
    if (e.act == SILU && !inputs[BUF_MAXNUM - 1].addr) return fail(ONE_ERR_BAD_ARG, "Conv: SILU needs the table in inputs[11]");
    one_ctx *ctx;
    if ((rc = default_ctx(&ctx)) != ONE_OK) return rc;
    cudaStream_t st = 0;   // legacy default stream: ordered after the caller's earlier work
    ws_reset(ctx);
    if (g.depthwise) {
        const float *aux;
        if ((rc = depthwise_aux(ctx, g, e, cfg, &aux, st)) != ONE_OK) return rc;
        rc = run_depthwise(g, e, reinterpret_cast<const float *>(inputs[0].addr), reinterpret_cast<const void *>(inputs[1].addr),
                           reinterpret_cast<const void *>(inputs[2].addr), aux, reinterpret_cast<const float *>(inputs[BUF_MAXNUM - 1].addr),
                           reinterpret_cast<float *>(outputs[0].addr), st);
        return rc != ONE_OK ? rc : finish_sync(ctx, st);
    }
    const int kind = e.int8 ? KIND_I8 : kind_of_prec(t_eval_prec);
    ConvPlan pl;
    plan_conv(g, kind, &pl, true);
    const long long M = (long long)g.N * g.OH * g.OW;
    if (conv_eval_scratch(g, e, pl) > ctx->ws_bytes)   // refused before anything is launched
        return fail(ONE_ERR_NOMEM, "Conv: this shape needs %zu bytes of scratch, the workspace holds %zu", conv_eval_scratch(g, e, pl), ctx->ws_bytes);
    const float inv_scale = e.int8 ? 1.0f / e.in_scale : 1.f;   // conv.c:943
    ConvIO io;
    memset(&io, 0, sizeof(io));
    cudaError_t ce;
    if (reads_reference_layout(pl)) {
        io.x = reinterpret_cast<const void *>(inputs[0].addr);
        io.x_nchw_f32 = 1;
        io.x_inv_scale = inv_scale;
    } else {
        void *xh = ws_alloc(ctx, (size_t)g.N * g.H * g.W * g.C * pl.es);
        if (!xh) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the NHWC input copy");
        ce = nchw_to_nhwc(reinterpret_cast<const float *>(inputs[0].addr), xh, g.N, g.C, g.H * g.W, pl.adt, 1, inv_scale, st);
        if (ce != cudaSuccess) return cuda_fail(ce, "nchw_to_nhwc");
        io.x = xh;
    }
    void *wp = ws_alloc(ctx, (size_t)g.OC * pl.w_pitch * pl.es);
    float *yh = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)M * g.OC * 4));
    if (!wp || !yh) return fail(ONE_ERR_NOMEM, "Conv: workspace too small (weights / NHWC output)");
    ce = pack_weights_for(g, pl, reinterpret_cast<const void *>(inputs[1].addr), wp, e.int8, st);
    if (ce != cudaSuccess) return cuda_fail(ce, "pack_conv_weight");
    io.w = wp;
    io.bias = e.has_bias ? reinterpret_cast<const void *>(inputs[2].addr) : nullptr;
    if (e.int8 && e.has_bias) {   // the kernel takes the int32 bias already cast to float
        float *bf = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)g.OC * 4));
        if (!bf) return fail(ONE_ERR_NOMEM, "Conv: workspace too small (bias)");
        if ((ce = cast_s32_f32(reinterpret_cast<const int *>(inputs[2].addr), bf, g.OC, st)) != cudaSuccess) return cuda_fail(ce, "cast_s32_f32");
        io.bias = bf;
    }
    io.lut = reinterpret_cast<const float *>(inputs[BUF_MAXNUM - 1].addr);
    std::vector<float> coeff;
    if (e.int8) {
        dequant_coeffs(cfg, g.OC, &coeff);
        float *cd = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)g.OC * 4));
        if (!cd) return fail(ONE_ERR_NOMEM, "Conv: workspace too small (coefficients)");
        if ((ce = cudaMemcpyAsync(cd, coeff.data(), (size_t)g.OC * 4, cudaMemcpyHostToDevice, st)) != cudaSuccess)
            return cuda_fail(ce, "coefficient upload");
        io.coeff = cd;
    }
    io.y = yh;
    io.out_mode = OUT_F32;
    if ((rc = run_conv(ctx, g, e, pl, io, nullptr, st)) != ONE_OK) return rc;
    ce = nhwc_to_nchw(yh, reinterpret_cast<float *>(outputs[0].addr), g.N, g.OC, g.OH * g.OW, DT_F32, st);
    if (ce != cudaSuccess) return cuda_fail(ce, "nhwc_to_nchw");
    return finish_sync(ctx, st);
}

extern "C" int one_cuda_gemm_eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs)
{
    if (!params || !params[1].addr || !params[4].addr) return fail(ONE_ERR_BAD_ARG, "Gemm: params[1] / params[4] descriptors are null");
    if (!inputs || !outputs || !inputs[0].addr || !inputs[1].addr || !inputs[2].addr || !outputs[0].addr)
        return fail(ONE_ERR_BAD_ARG, "Gemm: null tensor pointer");
    const OPERAND_S *a = reinterpret_cast<const OPERAND_S *>(params[1].addr);
    const OPERAND_S *y = reinterpret_cast<const OPERAND_S *>(params[4].addr);
    if (a->dim_num_of_shapes < 2 || a->dim_num_of_shapes > SHAPE_LEN || y->dim_num_of_shapes < 1 || y->dim_num_of_shapes > SHAPE_LEN)
        return fail(ONE_ERR_BAD_SHAPE, "Gemm: A needs at least 2 dims");
    // Only the last two dims of A are used and W is always read as [N][K] (gemm.c:30-55).
    const int M = a->shapes[a->dim_num_of_shapes - 2], K = a->shapes[a->dim_num_of_shapes - 1];
    const int N = y->shapes[y->dim_num_of_shapes - 1];
    if (M <= 0 || K <= 0 || N <= 0) return fail(ONE_ERR_BAD_SHAPE, "Gemm: non-positive dimension");
    one_ctx *ctx;
    int rc = default_ctx(&ctx);
    if (rc != ONE_OK) return rc;
    cudaStream_t st = 0;
    ws_reset(ctx);
    const int kind = kind_of_prec(t_eval_prec);
    const int es = kind_es(kind), Kp = round_up(K, 32 / es);
    void *ap = ws_alloc(ctx, (size_t)M * Kp * es);
    void *wp = ws_alloc(ctx, (size_t)N * Kp * es);
    if (!ap || !wp) return fail(ONE_ERR_NOMEM, "Gemm: workspace too small");
    cudaError_t ce = pack_rows(reinterpret_cast<const float *>(inputs[0].addr), ap, M, K, Kp, kind_dt(kind), st);
    if (ce == cudaSuccess) ce = pack_rows(reinterpret_cast<const float *>(inputs[1].addr), wp, N, K, Kp, kind_dt(kind), st);
    if (ce != cudaSuccess) return cuda_fail(ce, "pack_rows");
    rc = run_gemm(ctx, kind, ap, Kp, wp, Kp, M, N, K, 0, 0, 0, reinterpret_cast<void *>(outputs[0].addr), N, 0, OUT_F32,
                  reinterpret_cast<const float *>(inputs[2].addr), nullptr, pick_bn(N, M), st);
    if (rc != ONE_OK) return rc;
    return finish_sync(ctx, st);
}

// MatMul of two device tensors, A [batch..][M][K] x B [batch..][K][N] or a B shared by every batch
// (device/x86/MatMul/mat_mul.c:17-98).  Operand copies (A padded to the slab, B transposed to
// K-major) come from the context's workspace; everything is enqueued on `st`.
static int matmul_enqueue(one_ctx *ctx, int kind, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs,
                          cudaStream_t st, double *flops, double *bytes)
{
    MatmulShape s;
    int rc = parse_matmul(params, &s);
    if (rc != ONE_OK) return rc;
    if (!inputs || !outputs || !inputs[0].addr || !inputs[1].addr || !outputs[0].addr)
        return fail(ONE_ERR_BAD_ARG, "MatMul: null tensor pointer");
    ws_reset(ctx);
    const int es = kind_es(kind), Kp = round_up(s.K, 32 / es);
    const long long rowsA = (long long)s.batch * s.M;
    const void *A = reinterpret_cast<const void *>(inputs[0].addr);
    int a_pitch = s.K;
    cudaError_t ce = cudaSuccess;
    // fp32 rows whose pitch the tensor map accepts are read in place (the tensor core drops the
    // low mantissa bits of a tf32 operand itself)
    const bool a_in_place = kind == KIND_TF32 && (s.K * 4) % 16 == 0 && (inputs[0].addr & 15) == 0;
    const int nb = s.b_shared ? 1 : s.batch;
    // both operand copies are taken from the workspace before the first kernel is launched
    void *ap = a_in_place ? nullptr : ws_alloc(ctx, (size_t)rowsA * Kp * es);
    void *bp = ws_alloc(ctx, (size_t)nb * s.N * Kp * es);
    if ((!a_in_place && !ap) || !bp) return fail(ONE_ERR_NOMEM, "MatMul: workspace too small");
    if (!a_in_place) {
        ce = pack_rows(reinterpret_cast<const float *>(A), ap, rowsA, s.K, Kp, kind_dt(kind), st);
        if (ce != cudaSuccess) return cuda_fail(ce, "MatMul operand packing");
        A = ap; a_pitch = Kp;
    }
    ce = pack_transposed(reinterpret_cast<const float *>(inputs[1].addr), bp, nb, s.K, s.N, Kp, kind_dt(kind), st);
    if (ce != cudaSuccess) return cuda_fail(ce, "MatMul operand packing");
    void *out = reinterpret_cast<void *>(outputs[0].addr);
    if (s.b_shared)   // every batch shares B: one GEMM over batch*M rows
        rc = run_gemm(ctx, kind, A, a_pitch, bp, Kp, rowsA, s.N, s.K, 0, 0, 0, out, s.N, 0, OUT_F32, nullptr, nullptr, pick_bn(s.N, rowsA), st);
    else
        rc = run_gemm(ctx, kind, A, a_pitch, bp, Kp, s.M, s.N, s.K, s.batch, (long long)s.M * a_pitch, (long long)s.N * Kp, out, s.N,
                      (long long)s.M * s.N, OUT_F32, nullptr, nullptr, pick_bn(s.N, (long long)s.M * s.batch), st);
    if (flops) *flops = 2.0 * (double)rowsA * s.N * s.K;
    if (bytes) *bytes = ((double)rowsA * s.K + (double)nb * s.K * s.N + (double)rowsA * s.N) * 4.0;
    return rc;
}

extern "C" int one_cuda_matmul_eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs)
{
    MatmulShape s;   // descriptors are checked before anything touches the device
    int rc = parse_matmul(params, &s);
    if (rc != ONE_OK) return rc;
    if (!inputs || !outputs || !inputs[0].addr || !inputs[1].addr || !outputs[0].addr)
        return fail(ONE_ERR_BAD_ARG, "MatMul: null tensor pointer");
    one_ctx *ctx;
    if ((rc = default_ctx(&ctx)) != ONE_OK) return rc;
    cudaStream_t st = 0;
    const int kind = kind_of_prec(t_eval_prec);
    if ((rc = matmul_enqueue(ctx, kind, params, inputs, outputs, st, nullptr, nullptr)) != ONE_OK) return rc;
    return finish_sync(ctx, st);
}

extern "C" int one_cuda_matmul_async(one_ctx *ctx, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs,
                                     int flags, void *stream, double *flops, double *bytes)
{
    if (!ctx) return fail(ONE_ERR_BAD_ARG, "one_cuda_matmul_async: null context");
    const int prec = flags & ONE_PREC_MASK;
    if (!valid_prec(prec)) return fail(ONE_ERR_BAD_ARG, "unknown precision %d", prec);
    cudaStream_t st = stream ? reinterpret_cast<cudaStream_t>(stream) : ctx->stream;
    return matmul_enqueue(ctx, kind_of_prec(prec), params, inputs, outputs, st, flops, bytes);
}

// ============================================================================ prepared path
struct one_packed {
    int op;            // 0 Conv, 1 Gemm, 2 MatMul
    int flags;
    int kind;
    one_ctx *ctx;
    // Conv
    ConvGeom g;        // N is refreshed per call
    ConvGeom gp;       // the paired form actually launched when `paired`
    bool paired = false;
    ConvEpi e;
    ConvPlan pl;
    // Gemm / MatMul
    int M, K, N, Kp, b_shared, bn;
    // device-resident constants
    void *w = nullptr;
    void *bias = nullptr;
    float *coeff = nullptr;
    float *lut = nullptr;
    CUtensorMap tmB;
    bool tmB_valid = false;
    float q_inv_scale = 0.f;   // 1 / input_scale of the int8 consumer of outputs[1]
    double flops = 0, bytes = 0;
    char detail[160] = {0};    // shape and tile of the last evaluation
    int split_k = 0;           // this operator's split-K choice (0: the calling thread's setting)
};

static int upload(void **dst, const void *src, size_t bytes)
{
    cudaError_t e = cudaMalloc(dst, bytes ? bytes : 16);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc (prepare)");
    if (bytes && (e = cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail(e, "weight upload");
    return ONE_OK;
}

extern "C" int one_cuda_packed_release(one_packed *op)
{
    if (!op) return ONE_OK;
    cudaSetDevice(op->ctx->device);
    cudaFree(op->w); cudaFree(op->bias); cudaFree(op->coeff); cudaFree(op->lut);
    delete op;
    return ONE_OK;
}

extern "C" int one_cuda_packed_set_split(one_packed *op, int splits)
{
    if (!op || splits < 0 || splits > 64) return fail(ONE_ERR_BAD_ARG, "one_cuda_packed_set_split: split count must be 0 (default), 1 (never) or 2..64");
    op->split_k = splits;
    return ONE_OK;
}

namespace {
// The operator's own split-K choice overrides the calling thread's for the duration of one call.
struct ScopedSplit {
    int saved;
    explicit ScopedSplit(int v) : saved(t_split_k) { if (v) t_split_k = v; }
    ~ScopedSplit() { t_split_k = saved; }
};
}  // namespace

extern "C" int one_cuda_packed_detail(one_packed *op, char *buf, size_t cap)
{
    if (!op || !buf || !cap) return fail(ONE_ERR_BAD_ARG, "one_cuda_packed_detail: null argument");
    snprintf(buf, cap, "%s", op->detail);
    return ONE_OK;
}

extern "C" int one_cuda_packed_work(one_packed *op, double *flops, double *bytes)
{
    if (!op) return fail(ONE_ERR_BAD_ARG, "null operator");
    if (flops) *flops = op->flops;
    if (bytes) *bytes = op->bytes;
    return ONE_OK;
}

static int prepare_conv(one_packed *op, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, int prec, void **tmp)
{
    const CONV_CONFIG_S *cfg;
    int rc = parse_conv(params, &op->g, &op->e, &cfg);
    if (rc != ONE_OK) return rc;
    if (!inputs[1].addr || (op->e.has_bias && !inputs[2].addr)) return fail(ONE_ERR_BAD_ARG, "Conv prepare: null weight / bias");
    op->op = 0;
    if (op->g.depthwise) {
        // weights as they are (fp32, or int8 with the int32 bias and weight_aux), operating on the reference layout
        if (op->flags & ONE_LAYOUT_NHWC) return fail(ONE_ERR_UNSUPPORTED, "Conv prepare: depthwise runs on the reference layout (no ONE_LAYOUT_NHWC)");
        op->kind = op->e.int8 ? KIND_I8 : KIND_TF32;
        const ConvGeom &gd = op->g;
        if ((rc = upload(&op->w, reinterpret_cast<const void *>(inputs[1].addr), (size_t)gd.OC * gd.KH * gd.KW * (op->e.int8 ? 1 : 4))) != ONE_OK) return rc;
        if (op->e.has_bias && (rc = upload(&op->bias, reinterpret_cast<const void *>(inputs[2].addr), (size_t)gd.OC * 4)) != ONE_OK) return rc;
        if (op->e.int8 && (rc = upload(reinterpret_cast<void **>(&op->coeff), cfg->weight_aux, (size_t)gd.OC * 4)) != ONE_OK) return rc;
        if (op->e.act == SILU) {
            if (!inputs[BUF_MAXNUM - 1].addr) return fail(ONE_ERR_BAD_ARG, "Conv prepare: SILU needs the table in inputs[11]");
            if ((rc = upload(reinterpret_cast<void **>(&op->lut), reinterpret_cast<const void *>(inputs[BUF_MAXNUM - 1].addr), 8192 * 4)) != ONE_OK) return rc;
        }
        return ONE_OK;
    }
    op->kind = op->e.int8 ? KIND_I8 : kind_of_prec(prec);
    const bool resident_nhwc = (op->flags & ONE_LAYOUT_NHWC) && !(op->flags & ONE_IN_NCHW_F32);
    op->paired = resident_nhwc && pair_geometry(op->g, op->e, kind_es(op->kind), &op->gp);
    std::vector<float> wpair, bpair;
    const void *w_host = reinterpret_cast<const void *>(inputs[1].addr);
    const void *b_host = reinterpret_cast<const void *>(inputs[2].addr);
    if (op->paired) {
        pair_weights(reinterpret_cast<const float *>(w_host), op->g, &wpair);
        w_host = wpair.data();
        if (op->e.has_bias) {
            const float *b0 = reinterpret_cast<const float *>(b_host);
            bpair.assign(b0, b0 + op->g.OC);
            bpair.insert(bpair.end(), b0, b0 + op->g.OC);
            b_host = bpair.data();
        }
    }
    const ConvGeom &g = op->paired ? op->gp : op->g;   // the geometry that is planned, packed and launched
    plan_conv(g, op->kind, &op->pl, !(op->flags & ONE_LAYOUT_NHWC) || (op->flags & ONE_IN_NCHW_F32));
    const size_t welems = (size_t)g.OC * g.C * g.KH * g.KW;
    if ((rc = upload(tmp, w_host, op->e.int8 ? welems : welems * 4)) != ONE_OK) return rc;
    cudaError_t ce = cudaMalloc(&op->w, (size_t)g.OC * op->pl.w_pitch * op->pl.es);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaMalloc");
    ce = pack_weights_for(g, op->pl, *tmp, op->w, op->e.int8, 0);
    if (ce != cudaSuccess) return cuda_fail(ce, "pack_conv_weight");
    if (op->e.has_bias) {
        if (op->e.int8) {   // the kernel takes the int32 bias already cast to float (exact C cast)
            std::vector<float> bf(g.OC);
            const int *bi = reinterpret_cast<const int *>(inputs[2].addr);
            for (int i = 0; i < g.OC; ++i) bf[i] = (float)bi[i];
            if ((rc = upload(&op->bias, bf.data(), (size_t)g.OC * 4)) != ONE_OK) return rc;
        } else if ((rc = upload(&op->bias, b_host, (size_t)g.OC * 4)) != ONE_OK) return rc;
    }
    if (op->e.int8) {
        std::vector<float> coeff;
        dequant_coeffs(cfg, g.OC, &coeff);
        if ((rc = upload(reinterpret_cast<void **>(&op->coeff), coeff.data(), (size_t)g.OC * 4)) != ONE_OK) return rc;
    }
    if (op->e.act == SILU) {
        if (!inputs[BUF_MAXNUM - 1].addr) return fail(ONE_ERR_BAD_ARG, "Conv prepare: SILU needs the table in inputs[11]");
        if ((rc = upload(reinterpret_cast<void **>(&op->lut), reinterpret_cast<const void *>(inputs[BUF_MAXNUM - 1].addr), 8192 * 4)) != ONE_OK) return rc;
    }
    rc = make_tmap_tiled(&op->tmB, kind_tm(op->kind), op->w, op->pl.w_pitch, g.OC, 0, (uint64_t)op->pl.w_pitch * op->pl.es, 0,
                         op->pl.slab_elems, op->pl.cta2 ? op->pl.bn / 2 : op->pl.bn, op->pl.slab_bytes);
    if (rc == ONE_OK) op->tmB_valid = true;
    return rc;
}

static int prepare_gemm(one_packed *op, bool is_gemm, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, int prec, void **tmp)
{
    op->op = is_gemm ? 1 : 2;
    op->kind = kind_of_prec(prec);
    const int es = kind_es(op->kind);
    int rc;
    if (is_gemm) {
        if (!params[1].addr || !params[4].addr || !inputs[1].addr || !inputs[2].addr) return fail(ONE_ERR_BAD_ARG, "Gemm prepare: null descriptor / weight");
        const OPERAND_S *a = reinterpret_cast<const OPERAND_S *>(params[1].addr);
        const OPERAND_S *y = reinterpret_cast<const OPERAND_S *>(params[4].addr);
        if (a->dim_num_of_shapes < 2 || a->dim_num_of_shapes > SHAPE_LEN || y->dim_num_of_shapes < 1 || y->dim_num_of_shapes > SHAPE_LEN)
            return fail(ONE_ERR_BAD_SHAPE, "Gemm: A needs at least 2 dims");
        op->K = a->shapes[a->dim_num_of_shapes - 1];
        op->N = y->shapes[y->dim_num_of_shapes - 1];
    } else {
        MatmulShape s;
        if ((rc = parse_matmul(params, &s)) != ONE_OK) return rc;
        if (!s.b_shared)
            return fail(ONE_ERR_UNSUPPORTED, "MatMul prepare: B must be an initialiser shared by every batch; use one_cuda_matmul_eval for activation x activation");
        if (!inputs[1].addr) return fail(ONE_ERR_BAD_ARG, "MatMul prepare: null B");
        op->K = s.K; op->N = s.N;
    }
    op->b_shared = 1;
    if (op->K <= 0 || op->N <= 0) return fail(ONE_ERR_BAD_SHAPE, "non-positive dimension");
    op->Kp = round_up(op->K, 32 / es);
    {
        const OPERAND_S *a0 = reinterpret_cast<const OPERAND_S *>(params[1].addr);
        long long rows = 1;
        for (int i = 0; i < a0->dim_num_of_shapes - 1 && i < SHAPE_LEN; ++i) rows *= a0->shapes[i];
        op->bn = pick_bn(op->N, rows);
    }
    if ((rc = upload(tmp, reinterpret_cast<const void *>(inputs[1].addr), (size_t)op->K * op->N * 4)) != ONE_OK) return rc;
    cudaError_t ce = cudaMalloc(&op->w, (size_t)op->N * op->Kp * es);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaMalloc");
    ce = is_gemm ? pack_rows(reinterpret_cast<const float *>(*tmp), op->w, op->N, op->K, op->Kp, kind_dt(op->kind), 0)
                 : pack_transposed(reinterpret_cast<const float *>(*tmp), op->w, 1, op->K, op->N, op->Kp, kind_dt(op->kind), 0);
    if (ce != cudaSuccess) return cuda_fail(ce, "weight packing");
    // Gemm always has a bias; a MatMul has one when the following Add of a constant vector was folded in
    if ((is_gemm || inputs[2].addr) && (rc = upload(&op->bias, reinterpret_cast<const void *>(inputs[2].addr), (size_t)op->N * 4)) != ONE_OK) return rc;
    if (op->flags & ONE_FUSE_GELU) {
        if (!inputs[BUF_MAXNUM - 1].addr) return fail(ONE_ERR_BAD_ARG, "prepare: ONE_FUSE_GELU needs the table in inputs[11]");
        if ((rc = upload(reinterpret_cast<void **>(&op->lut), reinterpret_cast<const void *>(inputs[BUF_MAXNUM - 1].addr), 8192 * 4)) != ONE_OK) return rc;
    }
    const int slab_bytes = slab_for_bytes((long long)op->K * es);
    rc = make_tmap_tiled(&op->tmB, kind_tm(op->kind), op->w, op->K, op->N, 0, (uint64_t)op->Kp * es, 0, slab_bytes / es,
                         tile_cta2(op->bn) ? tile_bn(op->bn) / 2 : tile_bn(op->bn), slab_bytes);
    if (rc == ONE_OK) op->tmB_valid = true;
    return rc;
}

extern "C" int one_cuda_prepare(one_ctx *ctx, const char *op_type, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs,
                                int flags, one_packed **out)
{
    if (!ctx || !op_type || !params || !inputs || !out) return fail(ONE_ERR_BAD_ARG, "one_cuda_prepare: null argument");
    cudaError_t ce = cudaSetDevice(ctx->device);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
    const int prec = flags & ONE_PREC_MASK;
    if (!valid_prec(prec)) return fail(ONE_ERR_BAD_ARG, "unknown precision %d", prec);
    one_packed *op = new one_packed();
    op->ctx = ctx; op->flags = flags;
    void *tmp = nullptr;   // staging copy of the host weights
    int rc;
    if (!strcmp(op_type, "Conv")) rc = prepare_conv(op, params, inputs, prec, &tmp);
    else if (!strcmp(op_type, "Gemm")) rc = prepare_gemm(op, true, params, inputs, prec, &tmp);
    else if (!strcmp(op_type, "MatMul")) rc = prepare_gemm(op, false, params, inputs, prec, &tmp);
    else rc = fail(ONE_ERR_UNSUPPORTED, "one_cuda_prepare: operator type '%s' is not Conv, Gemm or MatMul", op_type);
    if (rc == ONE_OK && (ce = cudaDeviceSynchronize()) != cudaSuccess) rc = cuda_fail(ce, "prepare synchronise");
    if (tmp) cudaFree(tmp);
    if (rc != ONE_OK) {
        one_cuda_packed_release(op);
        return rc;
    }
    *out = op;
    return ONE_OK;
}

extern "C" int one_cuda_packed_set_requant(one_packed *op, float next_input_scale)
{
    if (!op || !(next_input_scale > 0.f)) return fail(ONE_ERR_BAD_ARG, "one_cuda_packed_set_requant: bad argument");
    op->q_inv_scale = 1.0f / next_input_scale;
    return ONE_OK;
}

extern "C" int one_cuda_eval_async(one_ctx *ctx, one_packed *op, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs,
                                   BUFFER_INFO_S *outputs, void *stream)
{
    if (!ctx || !op || !params || !inputs || !outputs) return fail(ONE_ERR_BAD_ARG, "one_cuda_eval_async: null argument");
    // a Conv may have no fp32 output at all when its int8 copy (outputs[ONE_SLOT_OUT_Q]) is all the consumer reads
    if (!inputs[0].addr || (!outputs[0].addr && !(op->op == 0 && outputs[ONE_SLOT_OUT_Q].addr)))
        return fail(ONE_ERR_BAD_ARG, "one_cuda_eval_async: null tensor pointer");
    cudaStream_t st = stream ? reinterpret_cast<cudaStream_t>(stream) : ctx->stream;
    ws_reset(ctx);
    ScopedSplit scoped_split(op->split_k);
    const bool nhwc = (op->flags & ONE_LAYOUT_NHWC) != 0;
    const bool bf16 = kind_is_16(op->kind);   // a 16-bit kind: bf16 or fp16
    if (op->op == 0) {
        if (!params[1].addr) return fail(ONE_ERR_BAD_ARG, "Conv: params[1] is null");
        const OPERAND_S *x = reinterpret_cast<const OPERAND_S *>(params[1].addr);
        ConvGeom g = op->g;
        g.N = x->shapes[0];
        if (g.N <= 0 || x->shapes[1] != g.C || x->shapes[2] != g.H || x->shapes[3] != g.W)
            return fail(ONE_ERR_BAD_SHAPE, "Conv: input descriptor changed since prepare");
        const long long M = (long long)g.N * g.OH * g.OW;
        ConvGeom gl = op->paired ? op->gp : g;   // the geometry launched (pixel pairs when the operator was paired)
        gl.N = g.N;
        if (M > 0x7fffffffLL) return fail(ONE_ERR_BAD_SHAPE, "Conv: too many output pixels");
        if (g.depthwise) {
            op->flops = 2.0 * (double)M * g.OC * g.KH * g.KW;   // host/ops/conv.h:170-172
            op->bytes = ((double)g.N * g.C * g.H * g.W + (double)M * g.OC) * 4.0;
            return run_depthwise(g, op->e, reinterpret_cast<const float *>(inputs[0].addr), op->w, op->bias, op->coeff, op->lut,
                                 reinterpret_cast<float *>(outputs[0].addr), st);
        }
        ConvIO io;
        memset(&io, 0, sizeof(io));
        io.w = op->w; io.bias = op->bias; io.coeff = op->coeff; io.lut = op->lut;
        const float inv_scale = op->e.int8 ? 1.0f / op->e.in_scale : 1.f;
        cudaError_t ce;
        int rc;
        const void *xin = reinterpret_cast<const void *>(inputs[0].addr);
        if (!nhwc) {
            // reference layout in and out: re-lay through the workspace
            if (reads_reference_layout(op->pl)) {
                io.x = xin; io.x_nchw_f32 = 1; io.x_inv_scale = inv_scale;
            } else {
                void *xh = ws_alloc(ctx, (size_t)g.N * g.H * g.W * g.C * op->pl.es);
                if (!xh) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the NHWC input copy");
                if ((ce = nchw_to_nhwc(reinterpret_cast<const float *>(xin), xh, g.N, g.C, g.H * g.W, op->pl.adt, 1, inv_scale, st)) != cudaSuccess)
                    return cuda_fail(ce, "nchw_to_nhwc");
                io.x = xh;
            }
            float *yh = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)M * g.OC * 4));
            if (!yh) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the NHWC output");
            io.y = yh; io.out_mode = OUT_F32;
            if ((rc = run_conv(ctx, g, op->e, op->pl, io, &op->tmB, st)) != ONE_OK) return rc;
            if ((ce = nhwc_to_nchw(yh, reinterpret_cast<float *>(outputs[0].addr), g.N, g.OC, g.OH * g.OW, DT_F32, st)) != cudaSuccess)
                return cuda_fail(ce, "nhwc_to_nchw");
        } else {
            // device-resident NHWC activations
            if (op->flags & ONE_IN_NCHW_F32) {
                // network input still in the reference layout: the explicit im2col reads it as it
                // is; the tensor-map paths get an NHWC copy in the operand type
                if (reads_reference_layout(op->pl)) {
                    io.x = xin; io.x_nchw_f32 = 1; io.x_inv_scale = inv_scale;
                } else {
                    void *xh = ws_alloc(ctx, (size_t)g.N * g.H * g.W * g.C * op->pl.es);
                    if (!xh) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the NHWC input copy");
                    if ((ce = nchw_to_nhwc(reinterpret_cast<const float *>(xin), xh, g.N, g.C, g.H * g.W, op->pl.adt, 1, inv_scale, st)) != cudaSuccess)
                        return cuda_fail(ce, "nchw_to_nhwc");
                    io.x = xh;
                }
            } else if (op->e.int8 && !(op->flags & ONE_IN_S8)) {
                // quantise the fp32 NHWC input for this layer (conv.c:961-973)
                if (op->pl.path == PATH_EXPLICIT) return fail(ONE_ERR_UNSUPPORTED, "Conv int8 NHWC fp32 input with C %% 32 != 0: feed NCHW or int8");
                int8_t *q = reinterpret_cast<int8_t *>(ws_alloc(ctx, (size_t)g.N * g.H * g.W * g.C));
                if (!q) return fail(ONE_ERR_NOMEM, "Conv: workspace too small for the quantised input");
                if ((ce = quantize_s8(reinterpret_cast<const float *>(xin), q, (long long)g.N * g.H * g.W * g.C, inv_scale, st)) != cudaSuccess)
                    return cuda_fail(ce, "quantize_s8");
                io.x = q;
            } else {
                io.x = xin;
            }
            io.y = reinterpret_cast<void *>(outputs[0].addr);
            io.out_mode = (bf16 && !(op->flags & ONE_OUT_F32)) ? kind_out16(op->kind) : ((op->flags & ONE_OUT_BF16) ? OUT_BF16 : OUT_F32);
            io.round_tf32 = io.out_mode == OUT_F32 && !op->e.int8;   // an fp32 activation may feed tf32 products
            if (op->flags & (ONE_FUSE_ADD_RELU | ONE_FUSE_ADD)) {
                if (!inputs[ONE_SLOT_RESIDUAL].addr) return fail(ONE_ERR_BAD_ARG, "Conv: fused add needs the residual in inputs[%d]", ONE_SLOT_RESIDUAL);
                io.residual = reinterpret_cast<const void *>(inputs[ONE_SLOT_RESIDUAL].addr);
                io.res_relu = (op->flags & ONE_FUSE_ADD_RELU) != 0;
            }
            if (outputs[ONE_SLOT_OUT_Q].addr) {
                io.out_q = reinterpret_cast<int8_t *>(outputs[ONE_SLOT_OUT_Q].addr);
                if (!(op->q_inv_scale > 0.f)) return fail(ONE_ERR_BAD_ARG, "Conv: outputs[1] given but one_cuda_packed_set_requant was not called");
                io.q_inv_scale = op->q_inv_scale;
            }
            if ((rc = run_conv(ctx, gl, op->e, op->pl, io, &op->tmB, st)) != ONE_OK) return rc;
        }
        snprintf(op->detail, sizeof(op->detail), "M=%lld N=%d K=%d %dx%d/%d C=%d@%dx%d %s tile=128x%d split=%d%s%s", M, g.OC, g.C * g.KH * g.KW, g.KH, g.KW,
                 g.sh, g.C, g.H, g.W, kind_name(op->kind), op->pl.bn, t_last_split,
                 op->paired ? " paired" : "", op->pl.cta2 ? " 2cta" : (op->pl.mh == 2 ? " 2half" : (op->pl.nw == 12 ? " 12w" : "")));
        op->flops = 2.0 * (double)M * g.OC * g.C * g.KH * g.KW;   // host/ops/conv.h:159-176
        const double aes = (op->flags & ONE_IN_S8) ? 1.0 : (op->e.int8 ? 4.0 : (nhwc && bf16 ? 2.0 : 4.0));
        const double yes = outputs[0].addr ? ((nhwc && ((bf16 && !(op->flags & ONE_OUT_F32)) || (op->flags & ONE_OUT_BF16))) ? 2.0 : 4.0) : 0.0;
        const double oes = yes + ((nhwc && outputs[ONE_SLOT_OUT_Q].addr) ? 1.0 : 0.0);
        // a folded Add brings its other operand: read once, in the output's element type (as the Gemm branch counts it)
        const double res = (op->flags & (ONE_FUSE_ADD_RELU | ONE_FUSE_ADD)) ? (double)M * g.OC * yes : 0.0;
        op->bytes = (double)g.N * g.C * g.H * g.W * aes + (double)g.OC * g.C * g.KH * g.KW * op->pl.es + g.OC * 4.0 +
                    (double)M * g.OC * oes + res;
        return ONE_OK;
    }
    // Gemm / MatMul with a prepared (shared) B
    const OPERAND_S *a = reinterpret_cast<const OPERAND_S *>(params[1].addr);
    if (!a || a->dim_num_of_shapes < 2 || a->dim_num_of_shapes > SHAPE_LEN) return fail(ONE_ERR_BAD_SHAPE, "A needs at least 2 dims");
    long long rows = a->shapes[a->dim_num_of_shapes - 2];
    if (op->op == 2 || (op->flags & ONE_LAYOUT_NHWC))   // MatMul folds every leading dim into M; so does a batched Gemm
        for (int i = 0; i < a->dim_num_of_shapes - 2; ++i) rows *= a->shapes[i];
    if (a->shapes[a->dim_num_of_shapes - 1] != op->K) return fail(ONE_ERR_BAD_SHAPE, "K changed since prepare");
    const int es = kind_es(op->kind);
    const void *A = reinterpret_cast<const void *>(inputs[0].addr);
    int a_pitch = op->K;
    const bool a_native = nhwc && ((op->K * es) % 16 == 0);   // activation already in the operand type
    if (!a_native) {
        void *ap = ws_alloc(ctx, (size_t)rows * op->Kp * es);
        if (!ap) return fail(ONE_ERR_NOMEM, "workspace too small for the A operand copy");
        cudaError_t ce = pack_rows(reinterpret_cast<const float *>(A), ap, rows, op->K, op->Kp, kind_dt(op->kind), st);
        if (ce != cudaSuccess) return cuda_fail(ce, "pack_rows");
        A = ap; a_pitch = op->Kp;
    }
    const int out_mode = (nhwc && bf16 && !(op->flags & ONE_OUT_F32)) ? kind_out16(op->kind) : OUT_F32;
    GemmEpi epi;
    if (op->flags & ONE_FUSE_GELU) {   // the Gelu table is looked up exactly like the SiLU one (gelu.c:22-38)
        epi.act = SILU;
        epi.lut = op->lut;
    }
    if (op->flags & ONE_FUSE_ADD) {
        if (!inputs[ONE_SLOT_RESIDUAL].addr) return fail(ONE_ERR_BAD_ARG, "fused add needs the residual in inputs[%d]", ONE_SLOT_RESIDUAL);
        epi.residual = reinterpret_cast<const void *>(inputs[ONE_SLOT_RESIDUAL].addr);
    }
    int rc = run_gemm(ctx, op->kind, A, a_pitch, op->w, op->Kp, rows, op->N, op->K, 0, 0, 0,
                      reinterpret_cast<void *>(outputs[0].addr), op->N, 0, out_mode, reinterpret_cast<const float *>(op->bias),
                      &op->tmB, op->bn, st, &epi);
    if (rc != ONE_OK) return rc;
    snprintf(op->detail, sizeof(op->detail), "M=%lld N=%d K=%d %s tile=128x%d split=%d%s", rows, op->N, op->K, kind_name(op->kind), tile_bn(op->bn),
             t_last_split, tile_cta2(op->bn) ? " 2cta" : (tile_mh(op->bn) == 2 ? " 2half" : (tile_nw(op->bn) == 12 ? " 12w" : "")));
    op->flops = 2.0 * (double)rows * op->N * op->K;
    op->bytes = (double)rows * op->K * (a_native ? es : 4) + (double)op->N * op->K * es +
                (double)rows * op->N * (out_is_16(out_mode) ? 2 : 4) * (epi.residual ? 2 : 1);
    return ONE_OK;
}

// ============================================================================ no-allocation Conv
// one_cuda_conv_eval_static: the drop-in Conv for callers that must not allocate device memory.
//
// Some hosts hand their whole device-memory budget to their own arena at start-up, or run inside
// a latency budget in which a cudaMalloc (which may serialise the whole device) is not acceptable,
// or embed this library in a sandbox whose allocator they do not control.  For them every byte
// of scratch this call needs -- the NHWC / space-to-depth / im2col copy of the input, the
// re-ordered weights, the NHWC output, the int8 constants and the status word -- comes out of one
// array that is part of the library image itself.  Every GPU that loads the library carries that
// array until the process exits, which is why it is kept modest (ONE_STATIC_SCRATCH_BYTES).
//
// The array's name is only meaningful to device code; on the host it is a stand-in, so the
// device address is fetched once per device with cudaGetSymbolAddress (with that device current)
// and every kernel receives that address.  The fetch happens in the first call on a device:
// make that first call before any stream capture is begun.  Every call synchronises `stream`
// before it returns (it reads the status word back), so the result is complete on return.
//
// All calls share the array and it keeps the previous call's bytes.  Only the status word has
// to start at zero and is cleared on the stream at the top of every call; everything else is
// fully overwritten before it is read.  Two calls on one device must not overlap: on the GPU
// (different streams) they would trample each other's scratch, and on the host (two threads)
// they would race on the bump offset that hands the array out.  Run them one after the other.
static __device__ __align__(256) unsigned char g_static_scratch[ONE_STATIC_SCRATCH_BYTES];

namespace {
struct StaticSlot {
    bool ready = false;
    one_ctx ctx;
};
StaticSlot g_static_slot[64];
std::mutex g_static_mu;

}  // namespace

extern "C" int one_cuda_conv_eval_static(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs,
                                         void *stream)
{
    ConvGeom g; ConvEpi e; const CONV_CONFIG_S *cfg;
    int rc = parse_conv(params, &g, &e, &cfg);
    if (rc != ONE_OK) return rc;
    if (!inputs || !outputs || !inputs[0].addr || !inputs[1].addr || !outputs[0].addr || (e.has_bias && !inputs[2].addr))
        return fail(ONE_ERR_BAD_ARG, "Conv: null tensor pointer");
    if (e.act == SILU && !inputs[BUF_MAXNUM - 1].addr) return fail(ONE_ERR_BAD_ARG, "Conv: SILU needs the table in inputs[11]");
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaGetDevice (no usable CUDA device: this backend has no CPU fallback)");
    if (dev < 0 || dev >= 64) return fail(ONE_ERR_BAD_ARG, "device index %d out of range", dev);
    StaticSlot &slot = g_static_slot[dev];
    {
        // once per device, with that device current: the device address behind the symbol
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!slot.ready) {
            void *ptr = nullptr;
            if ((ce = cudaGetSymbolAddress(&ptr, g_static_scratch)) != cudaSuccess) return cuda_fail(ce, "cudaGetSymbolAddress(static scratch)");
            slot.ctx.device = dev;
            slot.ctx.stream = nullptr;
            slot.ctx.status_dev = reinterpret_cast<unsigned int *>(ptr);           // first 256 bytes: status word
            slot.ctx.ws = reinterpret_cast<uint8_t *>(ptr) + 256;
            slot.ctx.ws_bytes = (size_t)ONE_STATIC_SCRATCH_BYTES - 256;
            slot.ctx.allow_split = false;   // the scratch this call takes is exactly what is counted below
            slot.ready = true;
        }
    }
    one_ctx *ctx = &slot.ctx;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (g.depthwise) {   // no scratch beyond the int8 weight_aux copy
        if ((ce = cudaMemsetAsync(ctx->status_dev, 0, sizeof(unsigned int), st)) != cudaSuccess) return cuda_fail(ce, "status clear");
        const float *aux;
        ws_reset(ctx);
        if ((rc = depthwise_aux(ctx, g, e, cfg, &aux, st)) != ONE_OK) return rc;
        rc = run_depthwise(g, e, reinterpret_cast<const float *>(inputs[0].addr), reinterpret_cast<const void *>(inputs[1].addr),
                           reinterpret_cast<const void *>(inputs[2].addr), aux, reinterpret_cast<const float *>(inputs[BUF_MAXNUM - 1].addr),
                           reinterpret_cast<float *>(outputs[0].addr), st);
        return rc != ONE_OK ? rc : finish_sync(ctx, st);
    }
    const int kind = e.int8 ? KIND_I8 : kind_of_prec(t_eval_prec);
    ConvPlan pl;
    plan_conv(g, kind, &pl, true);
    const long long M = (long long)g.N * g.OH * g.OW;
    // everything this call will carve out of the array, checked before anything is launched
    const size_t need = conv_eval_scratch(g, e, pl);
    if (need > ctx->ws_bytes)
        return fail(ONE_ERR_NOMEM, "Conv (static scratch): this shape needs %zu bytes of scratch, the built-in array holds %zu; use one_cuda_conv_eval or the prepared path",
                    need, ctx->ws_bytes);
    ws_reset(ctx);
    if ((ce = cudaMemsetAsync(ctx->status_dev, 0, sizeof(unsigned int), st)) != cudaSuccess) return cuda_fail(ce, "status clear");
    const float inv_scale = e.int8 ? 1.0f / e.in_scale : 1.f;
    ConvIO io;
    memset(&io, 0, sizeof(io));
    if (reads_reference_layout(pl)) {
        io.x = reinterpret_cast<const void *>(inputs[0].addr);
        io.x_nchw_f32 = 1;
        io.x_inv_scale = inv_scale;
    } else {
        void *xh = ws_alloc(ctx, (size_t)g.N * g.H * g.W * g.C * pl.es);
        if (!xh) return fail(ONE_ERR_NOMEM, "Conv (static scratch): NHWC input copy does not fit");
        if ((ce = nchw_to_nhwc(reinterpret_cast<const float *>(inputs[0].addr), xh, g.N, g.C, g.H * g.W, pl.adt, 1, inv_scale, st)) != cudaSuccess)
            return cuda_fail(ce, "nchw_to_nhwc");
        io.x = xh;
    }
    void *wp = ws_alloc(ctx, (size_t)g.OC * pl.w_pitch * pl.es);
    float *yh = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)M * g.OC * 4));
    if (!wp || !yh) return fail(ONE_ERR_NOMEM, "Conv (static scratch): weights / NHWC output do not fit");
    if ((ce = pack_weights_for(g, pl, reinterpret_cast<const void *>(inputs[1].addr), wp, e.int8, st)) != cudaSuccess)
        return cuda_fail(ce, "pack_conv_weight");
    io.w = wp;
    io.bias = e.has_bias ? reinterpret_cast<const void *>(inputs[2].addr) : nullptr;
    float coeff[ONE_WEIGHT_AUX_LEN];   // on the stack: no host allocation either
    if (e.int8) {
        if (e.has_bias) {
            float *bf = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)g.OC * 4));
            if (!bf) return fail(ONE_ERR_NOMEM, "Conv (static scratch): bias does not fit");
            if ((ce = cast_s32_f32(reinterpret_cast<const int *>(inputs[2].addr), bf, g.OC, st)) != cudaSuccess) return cuda_fail(ce, "cast_s32_f32");
            io.bias = bf;
        }
        for (int i = 0; i < g.OC; ++i) coeff[i] = cfg->weight_aux[i] * 1 / 127.0f;   // conv.c:1052
        float *cd = reinterpret_cast<float *>(ws_alloc(ctx, (size_t)g.OC * 4));
        if (!cd) return fail(ONE_ERR_NOMEM, "Conv (static scratch): coefficients do not fit");
        if ((ce = cudaMemcpyAsync(cd, coeff, (size_t)g.OC * 4, cudaMemcpyHostToDevice, st)) != cudaSuccess) return cuda_fail(ce, "coefficient upload");
        io.coeff = cd;
    }
    io.lut = reinterpret_cast<const float *>(inputs[BUF_MAXNUM - 1].addr);
    io.y = yh;
    io.out_mode = OUT_F32;
    if ((rc = run_conv(ctx, g, e, pl, io, nullptr, st)) != ONE_OK) return rc;
    if ((ce = nhwc_to_nchw(yh, reinterpret_cast<float *>(outputs[0].addr), g.N, g.OC, g.OH * g.OW, DT_F32, st)) != cudaSuccess)
        return cuda_fail(ce, "nhwc_to_nchw");
    return finish_sync(ctx, st);   // waits for the stream; `coeff` above stays alive until then
}
