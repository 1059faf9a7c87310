// prima.cpp_b200/csrc/layers.cu — the engine of the layer-list family (arch.h): a configuration file lists the layers, every layer has
// a sequence mixer (windowed attention with kept first tokens, a Mamba-2 state-space mixer, linear attention with a fixed decay per
// head, softmax attention over a low-rank latent, or a dual mixer: an attention branch beside a gated linear recurrence) and an optional
// feed-forward (tanh-GELU gated; clamped gated, dense or a routed mixture of experts), inside one of these layer frames: norms before and after every sublayer (FRAME_SANDWICH), or a grouped RMS norm
// before it with token shift and a depth average of all layer results (FRAME_PRENORM), or a layer norm with weight and bias on the
// sublayer's result only, scaled by one factor, with a learned position table on the embedding (FRAME_POSTNORM), or an RMS norm with one
// learned number before every sublayer, sublayer results times one factor, and a repeated block whose passes add the embedding output and
// a step vector (FRAME_PRERMS).  Weights are dense f32 / bf16 matrices.  It lives behind the same model object and C ABI as the k-quant transformer engine
// (engine.cu): pb200_model_set_tensor / _synth / _finalize / _free, sequence slots, device arg-max — and steps through the ragged
// batch step (pb200_batch_step) that the scheduler drives; the single-sequence entry points of the k-quant family answer PB200_ENOTSUP.
//
// State manager: every sequence slot owns one arena of constant size.  Per layer RUN (a layer inside a repeated block runs several
// times per token and each pass has its own state): attention -> K and V rows (positions below keep_first at their own row, later ones
// in a ring as long as the window), Mamba-2 -> the last taps-1 convolution inputs and the fp32 state [heads][state][vdim], decay
// attention -> the fp32 state [heads][dim][vdim], latent attention -> one row [latent | rotated key part] per position (a layer that
// reads another layer's latent has none of its own), token shift -> the normed input of the last token, dual mixer -> K and V rows, the
// last taps-1 convolution inputs of both branches and the recurrence's fp32 state.  A slot's arena is zeroed when it is handed out, so a
// reused slot starts like a new one; the token before a sequence's next one (bigram embedding) is kept per slot on the host.
//
// Precision: the residual stream, norms, attention scores / weights, recurrent state and everything that feeds the recurrence are
// fp32 in both compute types; with T_BF16 only the two operands of a dense product are bf16 (fp32 accumulation).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "arch.h"
#include "json.h"
#include "layers.h"
#include "model.h"

extern std::atomic<uint64_t> g_launches;

#define CK(expr)                  \
    do {                          \
        int _e = (int) (expr);    \
        if (_e != 0) return _e;   \
    } while (0)

namespace pb {

enum : int { MIX_ATTENTION = 0, MIX_MAMBA2 = 1, MIX_DECAY = 2, MIX_LATENT = 3, MIX_DUAL = 4 };
enum : int { FF_GELU = 0, FF_CLAMPED = 1, FF_MOE = 2, FF_RELU2 = 3 };   // FF_MOE: the expert form is MoeParams::act
enum : int { FRAME_SANDWICH = 0, FRAME_PRENORM = 1, FRAME_POSTNORM = 2, FRAME_PRERMS = 3 };
enum : int { ROUTE_SOFTMAX_TOP = 0, ROUTE_SIGMOID_GROUPS = 1, ROUTE_SIGMOID_PLAIN = 2 };
enum : int { REC_DELTA = 0, REC_HGRN2 = 1 };                 // recurrent branch of a dual mixer
enum : int { JOIN_SCALED_SUM = 0, JOIN_NORMED_MEAN = 1 };    // a * left + b * right through one output product, or the mean of the two normed results

struct DenseW {           // row-major [N][K] in the model's compute type
    void * data = nullptr;
    int64_t N = 0, K = 0;
    std::vector<uint8_t> filled;   // one flag per row block a checkpoint tensor fills (fused projections are filled by several tensors)
};
struct VecF {             // small fp32 parameter (norm weights, convolution taps, decay / step parameters)
    float * data = nullptr;
    int64_t n = 0;
    bool filled = false;
    std::vector<float> preset;   // non-empty: values the configuration fixes (decays, rotation frequencies); no checkpoint tensor fills it
    int n_parts = 0;             // > 0: several checkpoint tensors fill it, one flag each
    std::vector<uint8_t> parts;
};

// dual mixer: an attention branch (LLayer::att) and a gated linear recurrence side by side over the same input, ONE fused projection
struct DualMix {
    int rec = REC_DELTA, join = JOIN_SCALED_SUM;
    float left_scale = 1.f, right_scale = 1.f;
    int taps_l = 0, taps_r = 0, taps = 0;   // short convolution of the two branches (0: none); taps = the longer one, the shorter is padded with zero taps
    int qk_norm = QKN_NONE, rot_dims = 0, rot_layout = ROT_INTERLEAVED, v_rot = 0;
    int gate_mode = 1;                      // 1: a gate logit per head, 2: per output element
    GatedLinParams rp;
    // columns of the fused projection: left q | k | v, right q | k (HGRN2: forget logits) | v, then gates and per-head numbers; the first
    // conv_ch columns pass the convolution (the first conv_l of them without activation, the rest with SiLU)
    int c_q = 0, c_k = 0, c_v = 0, c_rq = 0, c_rk = 0, c_rv = 0, c_g = 0, c_rb = 0, c_ra = 0, c_rg = 0, cols = 0, conv_ch = 0, conv_l = 0;
};

struct LLayer {
    int kind = MIX_ATTENTION;
    AttnParams att;
    Mamba2Params ssm;
    int ff = 0;                        // 0: the layer has no feed-forward
    VecF norm1, norm1b, norm2, norm2b;
    DenseW qkvg, out;                  // attention: fused q | k | v | gate projection; `out` is the mixer's output projection of either kind
    DenseW in;                         // mamba2 input projection  z | x | B | C | dt
    VecF conv_w, conv_b, dt_bias, A_log, D, gnorm;
    DenseW gateup, down;               // feed-forward: fused gate | up
    int ff_kind = FF_GELU;
    float ff_limit = 0.f;              // FF_CLAMPED
    // decay attention (qkvg: fused q | k | v | gate with a gate logit per output element)
    DecayAttnParams dec;
    int dec_norm_groups = 1;           // output norm: 1 = all heads together, heads = every head by itself
    bool dec_norm_weight = false;
    int dec_gate_act = 0;              // 0 sigmoid, 1 silu
    VecF decay, onorm;
    // latent attention (lproj: fused dq | gate | dkv)
    LatentParams lat;
    int kv_from = -1;                  // >= 0: the layer whose latent cache this one reads
    DenseW lproj, uq, uk, uv;
    VecF dq_norm, dkv_norm, rot_freq;
    // mixture of experts: e_gateup [experts][2 ff][width], e_down [experts][width][ff]; a shared expert beside them (shared_ff > 0)
    MoeParams moe;
    DenseW e_gateup, e_down, s_gateup, s_down;
    VecF router, router_b;
    int shared_ff = 0;
    float shared_limit = 0.f;
    // FRAME_PRENORM
    VecF shift, dwa;
    // FRAME_POSTNORM: biases of the two norms
    VecF norm1_bias, norm2_bias;
    // attention: RMS norm of every query / key head with a weight [dim] all heads share
    bool qk_norm = false;
    VecF q_norm, k_norm;
    // mixture of experts: form of the router; the shared expert's per-token gate vector [width] (ROUTE_SIGMOID_GROUPS)
    int route = ROUTE_SOFTMAX_TOP;
    VecF shared_gate;
    // dual mixer (qkvg: the fused projection of both branches; out: the output product over [left | right], or the left one; out_r: the right one)
    DualMix dual;
    DenseW out_r;
    VecF dconv_w, vrot_freq, f_bias, f_lower, join_wl, join_wr;   // rot_freq, q_norm, k_norm, A_log, dt_bias, onorm are shared with the other mixers
};

struct LRun {
    int layer = 0;
    int pass = -1;            // >= 0: this run opens pass `pass` of the repeated block (input mix + step vector come first)
    int64_t state_off = 0;    // floats from the slot's arena base (a latent layer that reads another layer's cache: that layer's offset)
    int64_t shift_off = -1;   // token-shift state [width]
};

// where a checkpoint tensor goes
struct TensorPlace {
    DenseW * mat = nullptr;   // rows [row0, row0 + rows) of a matrix, columns [col0, col0 + cols) (col0 == 0 and cols == K: whole rows) ...
    int64_t row0 = 0, rows = 0, cols = 0, col0 = 0;
    int part = 0;             // index into mat->filled / vec->parts
    VecF * vec = nullptr;     // ... or a whole fp32 vector of n elements ...
    int64_t n = 0;
    // ... or (vrows > 0) a tensor [vrows][vcols] (n = vrows * vcols) placed at element v0 + r * vld + c, `repeat` copies vrep elements apart:
    // a block of a vector several tensors fill, a short convolution right-aligned in longer taps, a weight all heads share, one number for all
    int64_t v0 = 0, vrows = 0, vcols = 0, vld = 0, repeat = 1, vrep = 0;
};

struct LayerList {
    const ArchEntry * arch = nullptr;
    int ctype = T_BF16;       // compute type: operand type of the dense products
    int frame = FRAME_SANDWICH;
    int norm_groups = 1;      // FRAME_PRENORM: groups of the RMS norm
    int width = 0, vocab = 0;
    float eps = 1e-6f, logit_scale = 1.f;
    std::vector<LLayer> layers;
    std::vector<LRun> runs;
    // repeated block
    int loop_start = 0, loop_stop = 0, loop_times = 0;
    DenseW loop_in;
    VecF loop_step;
    DenseW embed, head;
    VecF final_norm;
    // FRAME_POSTNORM
    DenseW pos_table;         // learned position vectors [max_pos][width], added to the embedding
    int max_pos = 0;
    VecF final_norm_bias;
    float resid_mult = 1.f;   // factor on every normed sublayer result (FRAME_PRERMS: on every sublayer result)
    // FRAME_PRERMS: embedding factor, hashed bigram table [buckets + 1][width] (buckets == 0: none), the token before each slot's next one
    float embed_scale = 1.f;
    BigramParams bigram;
    DenseW bigram_table;
    std::vector<int32_t> seq_prev;
    float logit_softcap = 0.f;   // > 0: logits <- cap * tanh(logits / cap)
    // state manager
    int n_ctx = 0, n_seq = 0;
    bool ctx_limited = false;       // some cache holds every position: a sequence cannot outgrow n_ctx
    int64_t slot_floats = 0;
    float * state = nullptr;
    std::vector<int32_t> seq_len;   // -1: free
    // batch scratch (grown on demand)
    int capT = 0, capW = 0;
    float *x = nullptr, *x0 = nullptr, *xalt = nullptr, *big = nullptr, *msub = nullptr, *xbc = nullptr, *yssm = nullptr, *logits = nullptr;
    void *act = nullptr, *act2 = nullptr, *actw = nullptr;
    // FRAME_PRENORM and its mixers: results of all layers [layers + 1][capT][width]; further fp32 and operand-type scratch
    float *hist = nullptr, *big2 = nullptr, *big3 = nullptr, *big4 = nullptr, *krb = nullptr;
    float * lat_part = nullptr;     // partial results of the split decode attention kernels: latent [entries][splits][heads][kv_rank + 2], windowed [entries][heads][splits][vdim + 2]
    size_t lat_part_cap = 0;
    // mixture of experts: pairs (token, choice)
    int32_t *moe_idx = nullptr, *moe_perm = nullptr, *moe_row_of = nullptr, *moe_count = nullptr, *moe_start = nullptr, *moe_count_host = nullptr;
    float *moe_wt = nullptr, *moe_gu = nullptr, *moe_ds = nullptr, *moe_sg = nullptr;
    void *moe_y = nullptr, *moe_hs = nullptr;
    int32_t *meta_dev = nullptr, *meta_host = nullptr, *greedy_dev = nullptr, *greedy_host = nullptr;
    float * logits_host = nullptr;
    size_t meta_cap = 0, logits_host_cap = 0;
    std::vector<void *> scratch;
    // white-box tap: residual stream after every layer run of the last batch
    bool tap_on = false;
    float * tap = nullptr;
    int64_t tap_floats = 0, tap_cap = 0;
    int tap_T = 0;
    int64_t weight_bytes = 0;
    // per-category device time of the last batch step (bench): CUDA events around every launch while prof_on
    bool prof_on = false;
    std::vector<cudaEvent_t> prof_ev;
    std::vector<int> prof_cat;
    float prof_ms[10] = {0};
    // decode steps replayed as CUDA graphs, one per (entries, wanted rows); the batch's metadata lives at fixed device addresses
    struct StepGraph { cudaGraphExec_t exec = nullptr; int seen = 0; uint64_t launches = 0; };
    std::map<uint64_t, StepGraph> graphs;
    // a dual mixer's recurrent branch runs on a second stream beside the attention branch (fork after the token preparation, join before the
    // branches meet); the pair of events is capturable, so a replayed decode graph keeps the two branches side by side
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    std::vector<int> rows_tmp;      // logits row of the caller (or -(entry+1) for a greedy row) per wanted row of the last sub-batch
};

// ---------------------------------------------------------------------------------------------------------------
// Vamidra: configuration keys and tensor names
static int vamidra_configure(const Json & cfg, LayerList & ll, std::string & err) {
    ll.width = (int) cfg.integer("width", 0);
    ll.vocab = (int) cfg.integer("vocab", 0);
    ll.logit_scale = (float) cfg.number("logit_scale", 1.0);
    if (const Json * nrm = cfg.get("norm")) ll.eps = (float) nrm->number("eps", 1e-6);
    const Json * layers = cfg.get("layers");
    if (ll.width <= 0 || ll.vocab <= 0 || !layers || layers->kind != Json::ARR || layers->arr.empty()) { err = "width, vocab and layers are required"; return PB200_EINVAL; }
    for (const Json & jl : layers->arr) {
        LLayer L;
        const std::string type = jl.string("type");
        const Json * mx = jl.get("mixer");
        if (!mx || mx->kind != Json::OBJ) { err = "layer without mixer"; return PB200_EINVAL; }
        if (type == "attention") {
            L.kind = MIX_ATTENTION;
            AttnParams & a = L.att;
            a.heads = (int) mx->integer("heads", 0);
            a.kv_heads = (int) mx->integer("kv_heads", a.heads);
            a.dim = (int) mx->integer("dim", 0);
            a.vdim = (int) mx->integer("vdim", a.dim);
            a.scale = (float) mx->number("scale", a.dim > 0 ? 1.0 / std::sqrt((double) a.dim) : 1.0);
            a.softcap = (float) mx->number("softcap", 0.0);
            a.window = 0;
            a.keep_first = 0;
            if (const Json * mk = mx->get("mask")) {
                if (mk->kind == Json::OBJ) {
                    a.window = (int) std::min<long long>(mk->integer("size", 0), 1 << 30);
                    a.keep_first = (int) std::min<long long>(std::max<long long>(mk->integer("keep_first", 0), 0), 1 << 30);
                }
            }
            if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.dim <= 0 || a.vdim <= 0 || a.vdim > 256) { err = "attention sizes"; return PB200_EINVAL; }
        } else if (type == "mamba2") {
            L.kind = MIX_MAMBA2;
            Mamba2Params & p = L.ssm;
            p.heads = (int) mx->integer("heads", 0);
            p.vdim = (int) mx->integer("vdim", 0);
            p.state = (int) mx->integer("state", 0);
            p.groups = (int) mx->integer("groups", 1);
            p.conv = (int) mx->integer("conv", 1);
            p.norm_groups = (int) mx->integer("norm_groups", 1);
            if (p.heads <= 0 || p.vdim <= 0 || p.state <= 0 || p.groups <= 0 || p.heads % p.groups || p.conv < 1 || p.norm_groups <= 0 ||
                (p.heads * p.vdim) % p.norm_groups) { err = "mamba2 sizes"; return PB200_EINVAL; }
        } else {
            err = "unknown layer type '" + type + "'";
            return PB200_ENOTSUP;
        }
        const Json * mlp = jl.get("mlp");
        if (mlp && mlp->kind == Json::OBJ) {
            const std::string kind = mlp->string("kind", "dense");
            if (kind != "dense") { err = "unknown feed-forward kind '" + kind + "'"; return PB200_ENOTSUP; }
            L.ff = (int) mlp->integer("ff", 0);
            if (L.ff <= 0) { err = "feed-forward size"; return PB200_EINVAL; }
        }
        ll.layers.push_back(std::move(L));
    }
    const int nl = (int) ll.layers.size();
    ll.loop_times = 0;
    if (const Json * lp = cfg.get("loop")) {
        if (lp->kind == Json::OBJ) {
            ll.loop_start = (int) lp->integer("start", 0);
            ll.loop_stop = (int) lp->integer("stop", 0);
            ll.loop_times = (int) lp->integer("times", 1);
            if (ll.loop_start < 0 || ll.loop_stop > nl || ll.loop_start >= ll.loop_stop || ll.loop_times < 1) { err = "loop range"; return PB200_EINVAL; }
        }
    }
    // order of layer runs: layers before the block once, the block `times` times in a row, the rest once
    for (int i = 0; i < nl;) {
        if (ll.loop_times > 0 && i == ll.loop_start) {
            for (int t = 0; t < ll.loop_times; t++)
                for (int k = ll.loop_start; k < ll.loop_stop; k++) {
                    LRun r;
                    r.layer = k;
                    r.pass = k == ll.loop_start ? t : -1;
                    ll.runs.push_back(r);
                }
            i = ll.loop_stop;
        } else {
            LRun r;
            r.layer = i++;
            ll.runs.push_back(r);
        }
    }
    return 0;
}

static bool vamidra_resolve(LayerList & ll, const std::string & name, TensorPlace & o) {
    const int64_t W = ll.width;
    auto mat = [&](DenseW & m, int64_t row0, int64_t rows, int64_t cols, int part) { o.mat = &m; o.row0 = row0; o.rows = rows; o.cols = cols; o.part = part; return true; };
    auto vec = [&](VecF & v, int64_t n) { o.vec = &v; o.n = n; return true; };
    if (name == "embed") return mat(ll.embed, 0, ll.vocab, W, 0);
    if (name == "head") return mat(ll.head, 0, ll.vocab, W, 0);
    if (name == "final.norm") return vec(ll.final_norm, W);
    if (name == "loop.in") return ll.loop_times > 0 && mat(ll.loop_in, 0, W, 2 * W, 0);
    if (name == "loop.step") return ll.loop_times > 0 && vec(ll.loop_step, (int64_t) ll.loop_times * W);
    int il = -1, used = 0;
    if (sscanf(name.c_str(), "l%d.%n", &il, &used) != 1 || used <= 0 || il < 0 || il >= (int) ll.layers.size()) return false;
    LLayer & L = ll.layers[il];
    const std::string w = name.substr((size_t) used);
    if (w == "norm1") return vec(L.norm1, W);
    if (w == "norm1b") return vec(L.norm1b, W);
    if (L.ff > 0) {
        if (w == "norm2") return vec(L.norm2, W);
        if (w == "norm2b") return vec(L.norm2b, W);
        if (w == "mlp.gate") return mat(L.gateup, 0, L.ff, W, 0);
        if (w == "mlp.up") return mat(L.gateup, L.ff, L.ff, W, 1);
        if (w == "mlp.down") return mat(L.down, 0, W, L.ff, 0);
    }
    if (L.kind == MIX_ATTENTION) {
        const AttnParams & a = L.att;
        const int64_t QD = (int64_t) a.heads * a.dim, KD = (int64_t) a.kv_heads * a.dim, VD = (int64_t) a.kv_heads * a.vdim;
        if (w == "mix.q") return mat(L.qkvg, 0, QD, W, 0);
        if (w == "mix.k") return mat(L.qkvg, QD, KD, W, 1);
        if (w == "mix.v") return mat(L.qkvg, QD + KD, VD, W, 2);
        if (w == "mix.g") return mat(L.qkvg, QD + KD + VD, a.heads, W, 3);
        if (w == "mix.o") return mat(L.out, 0, W, (int64_t) a.heads * a.vdim, 0);
    } else {
        const Mamba2Params & p = L.ssm;
        if (w == "mix.in") return mat(L.in, 0, mamba2_in_cols(p), W, 0);
        if (w == "mix.conv") return vec(L.conv_w, (int64_t) mamba2_conv_channels(p) * p.conv);
        if (w == "mix.conv.b") return vec(L.conv_b, mamba2_conv_channels(p));
        if (w == "mix.dt_bias") return vec(L.dt_bias, p.heads);
        if (w == "mix.A_log") return vec(L.A_log, p.heads);
        if (w == "mix.D") return vec(L.D, p.heads);
        if (w == "mix.norm") return vec(L.gnorm, mamba2_inner(p));
        if (w == "mix.o") return mat(L.out, 0, W, mamba2_inner(p), 0);
    }
    return false;
}

// ---------------------------------------------------------------------------------------------------------------
// Mumizen: configuration keys and tensor names.  Pre-norm layers (RMS norm in groups), token shift on the mixer's input, depth average
// after every layer; mixers "lightning" / "retention" (decay attention) and "latent_attention"; clamped gated feed-forward, dense or "moe".
static int clamped_ff_config(const Json & jm, int & ff, float & limit, std::string & err) {
    ff = (int) jm.integer("ff", 0);
    limit = (float) jm.number("limit", 0.0);
    if (ff <= 0 || !(limit > 0.f)) { err = "feed-forward size / limit"; return PB200_EINVAL; }
    return 0;
}
// rotation frequencies with the long-context blend: below turn-count `fast` per original context a pair keeps its frequency, above
// `slow` it is divided by `factor`, linear in the pair index between; cos and sin then carry 0.1 ln(factor) + 1
static void rotary_table(const Json & rot, int dims, std::vector<float> & freq, float & mag) {
    const double base = rot.number("base", 10000.0);
    const int half = dims / 2;
    freq.assign((size_t) std::max(half, 1), 0.f);
    mag = 1.f;
    const Json * sc = rot.get("scaling");
    const bool scaled = sc && sc->kind == Json::OBJ;
    double lo = 0, hi = 0, factor = 1;
    if (scaled) {
        factor = sc->number("factor", 1.0);
        const double orig = sc->number("original", 1.0), fast = sc->number("fast", 32.0), slow = sc->number("slow", 1.0);
        auto turn_dim = [&](double turns) { return dims * std::log(orig / (2.0 * M_PI * turns)) / (2.0 * std::log(base)); };
        lo = std::max(std::floor(turn_dim(fast)), 0.0);
        hi = std::min(std::ceil(turn_dim(slow)), (double) dims - 1.0);
        mag = (float) (0.1 * std::log(factor) + 1.0);
    }
    for (int i = 0; i < half; i++) {
        const double f = std::pow(base, -2.0 * i / dims);
        double v = f;
        if (scaled) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            v = f / factor * ramp + f * (1.0 - ramp);
        }
        freq[(size_t) i] = (float) v;
    }
}

static int mumizen_configure(const Json & cfg, LayerList & ll, std::string & err) {
    ll.frame = FRAME_PRENORM;
    ll.width = (int) cfg.integer("width", 0);
    ll.vocab = (int) cfg.integer("vocab", 0);
    ll.logit_scale = 1.f;
    ll.norm_groups = 1;
    if (const Json * nrm = cfg.get("norm")) { ll.eps = (float) nrm->number("eps", 1e-6); ll.norm_groups = (int) nrm->integer("groups", 1); }
    const Json * layers = cfg.get("layers");
    if (ll.width <= 0 || ll.vocab <= 0 || !layers || layers->kind != Json::ARR || layers->arr.empty()) { err = "width, vocab and layers are required"; return PB200_EINVAL; }
    if (ll.norm_groups <= 0 || ll.norm_groups > 64 || ll.width % ll.norm_groups) { err = "norm groups"; return PB200_EINVAL; }
    for (const Json & jl : layers->arr) {
        LLayer L;
        const std::string type = jl.string("type");
        const Json * mx = jl.get("mixer");
        if (!mx || mx->kind != Json::OBJ) { err = "layer without mixer"; return PB200_EINVAL; }
        const int il = (int) ll.layers.size();
        if (type == "lightning" || type == "retention") {
            L.kind = MIX_DECAY;
            DecayAttnParams & d = L.dec;
            d.heads = (int) mx->integer("heads", 0);
            d.dim = (int) mx->integer("dim", 0);
            d.vdim = (int) mx->integer("vdim", d.dim);
            const Json * dc = mx->get("decay");
            if (d.heads <= 0 || d.dim <= 0 || d.vdim <= 0 || !dc || dc->kind != Json::ARR || (int) dc->arr.size() != d.heads) { err = type + " sizes / decay"; return PB200_EINVAL; }
            for (const Json & v : dc->arr) L.decay.preset.push_back((float) v.num);
            if (type == "lightning") {   // SiLU on q, k, v; all heads normed together with a weight; sigmoid gate
                d.act = 1; d.k_scale = 1.f;
                L.dec_norm_groups = 1; L.dec_norm_weight = true; L.dec_gate_act = 0;
            } else {                     // plain q, k, v with k / sqrt(dim); every head by its own root mean square, no weight; SiLU gate
                d.act = 0; d.k_scale = (float) (1.0 / std::sqrt((double) d.dim));
                L.dec_norm_groups = d.heads; L.dec_norm_weight = false; L.dec_gate_act = 1;
            }
        } else if (type == "latent_attention") {
            L.kind = MIX_LATENT;
            LatentParams & a = L.lat;
            a.heads = (int) mx->integer("heads", 0);
            a.dim = (int) mx->integer("dim", 0);
            a.rot_dim = (int) mx->integer("rot_dim", 0);
            a.vdim = (int) mx->integer("vdim", a.dim);
            a.kv_rank = (int) mx->integer("kv_rank", 0);
            a.q_rank = (int) mx->integer("q_rank", 0);
            a.scale = (float) mx->number("scale", a.dim + a.rot_dim > 0 ? 1.0 / std::sqrt((double) (a.dim + a.rot_dim)) : 1.0);
            a.rot_dims = 0;
            const Json * rot = mx->get("rot");
            if (rot && rot->kind == Json::OBJ) {
                a.rot_dims = (int) rot->integer("dims", a.rot_dim);
                if (a.rot_dims < 0 || a.rot_dims > a.rot_dim || a.rot_dims % 2) { err = "rotated dimensions"; return PB200_EINVAL; }
                rotary_table(*rot, a.rot_dims, L.rot_freq.preset, a.rot_mag);
            } else {
                L.rot_freq.preset.assign(1, 0.f);
            }
            const Json * from = mx->get("kv_from");
            a.own_kv = 1;
            if (from && from->kind == Json::NUM) {
                L.kv_from = (int) from->num;
                a.own_kv = 0;
                if (L.kv_from < 0 || L.kv_from >= il) { err = "kv_from must name an earlier layer"; return PB200_EINVAL; }
                const LLayer & S = ll.layers[(size_t) L.kv_from];
                if (S.kind != MIX_LATENT || !S.lat.own_kv || S.lat.kv_rank != a.kv_rank || S.lat.rot_dim != a.rot_dim) { err = "kv_from: the named layer has no latent cache of this shape"; return PB200_EINVAL; }
            }
            if (a.heads <= 0 || a.dim < 0 || a.rot_dim < 0 || a.dim + a.rot_dim <= 0 || a.vdim <= 0 || a.kv_rank <= 0 || a.q_rank <= 0 || a.kv_rank > 512 ||
                a.vdim > 512) { err = "latent attention sizes"; return PB200_EINVAL; }
        } else {
            err = "unknown layer type '" + type + "'";
            return PB200_ENOTSUP;
        }
        const Json * mlp = jl.get("mlp");
        if (mlp && mlp->kind == Json::OBJ) {
            const std::string kind = mlp->string("kind", "dense");
            if (kind == "dense") {
                L.ff_kind = FF_CLAMPED;
                int rc = clamped_ff_config(*mlp, L.ff, L.ff_limit, err);
                if (rc) return rc;
            } else if (kind == "moe") {
                L.ff_kind = FF_MOE;
                const Json * ex = mlp->get("expert"), * ro = mlp->get("router"), * sh = mlp->get("shared");
                if (!ex || ex->kind != Json::OBJ || !ro || ro->kind != Json::OBJ) { err = "moe needs expert and router"; return PB200_EINVAL; }
                int rc = clamped_ff_config(*ex, L.moe.ff, L.moe.limit, err);
                if (rc) return rc;
                L.ff = L.moe.ff;
                L.moe.experts = (int) ro->integer("experts", 0);
                L.moe.top = (int) ro->integer("top", 0);
                if (L.moe.experts <= 0 || L.moe.top <= 0 || L.moe.top > L.moe.experts || L.moe.top > 32 || L.moe.experts > 4096) { err = "router sizes"; return PB200_EINVAL; }
                if (sh && sh->kind == Json::OBJ) {
                    rc = clamped_ff_config(*sh, L.shared_ff, L.shared_limit, err);
                    if (rc) return rc;
                }
            } else {
                err = "unknown feed-forward kind '" + kind + "'";
                return PB200_ENOTSUP;
            }
        }
        ll.layers.push_back(std::move(L));
    }
    for (int i = 0; i < (int) ll.layers.size(); i++) {
        LRun r;
        r.layer = i;
        ll.runs.push_back(r);
    }
    return 0;
}

static bool mumizen_resolve(LayerList & ll, const std::string & name, TensorPlace & o) {
    const int64_t W = ll.width;
    auto mat = [&](DenseW & m, int64_t row0, int64_t rows, int64_t cols, int part) { o.mat = &m; o.row0 = row0; o.rows = rows; o.cols = cols; o.part = part; return true; };
    auto vec = [&](VecF & v, int64_t n) { o.vec = &v; o.n = n; return true; };
    if (name == "embed") return mat(ll.embed, 0, ll.vocab, W, 0);
    if (name == "head") return mat(ll.head, 0, ll.vocab, W, 0);
    if (name == "final.norm") return vec(ll.final_norm, W);
    int il = -1, used = 0;
    if (sscanf(name.c_str(), "l%d.%n", &il, &used) != 1 || used <= 0 || il < 0 || il >= (int) ll.layers.size()) return false;
    LLayer & L = ll.layers[(size_t) il];
    const std::string w = name.substr((size_t) used);
    if (w == "norm1") return vec(L.norm1, W);
    if (w == "shift") return vec(L.shift, W);
    if (w == "dwa") return vec(L.dwa, il + 2);
    // a clamped gated unit `pre`gate / up / down inside fused matrices: gate | up rows at gu_row0, down rows at d_row0
    auto glu = [&](const std::string & leaf, DenseW & gu, DenseW & dn, int64_t ff, int64_t gu_row0, int64_t d_row0, int part0) {
        if (leaf == "gate") return mat(gu, gu_row0, ff, W, part0);
        if (leaf == "up") return mat(gu, gu_row0 + ff, ff, W, part0 + 1);
        if (leaf == "down") return mat(dn, d_row0, W, ff, part0 / 2);
        return false;
    };
    if (L.ff > 0 && w == "norm2") return vec(L.norm2, W);
    if (L.ff > 0 && w.compare(0, 4, "mlp.") == 0) {
        const std::string f = w.substr(4);
        if (L.ff_kind == FF_CLAMPED) return glu(f, L.gateup, L.down, L.ff, 0, 0, 0);
        if (f == "router") { o.vec = &L.router; o.n = (int64_t) L.moe.experts * W; return true; }
        if (f == "router.b") return vec(L.router_b, L.moe.experts);
        if (f.compare(0, 7, "shared.") == 0) return L.shared_ff > 0 && glu(f.substr(7), L.s_gateup, L.s_down, L.shared_ff, 0, 0, 0);
        int e = -1, u2 = 0;
        if (sscanf(f.c_str(), "e%d.%n", &e, &u2) == 1 && u2 > 0 && e >= 0 && e < L.moe.experts)
            return glu(f.substr((size_t) u2), L.e_gateup, L.e_down, L.moe.ff, (int64_t) e * 2 * L.moe.ff, (int64_t) e * W, 2 * e);
        return false;
    }
    if (L.kind == MIX_DECAY) {
        const int64_t QD = (int64_t) L.dec.heads * L.dec.dim, VD = (int64_t) L.dec.heads * L.dec.vdim;
        if (w == "mix.q") return mat(L.qkvg, 0, QD, W, 0);
        if (w == "mix.k") return mat(L.qkvg, QD, QD, W, 1);
        if (w == "mix.v") return mat(L.qkvg, 2 * QD, VD, W, 2);
        if (w == "mix.g") return mat(L.qkvg, 2 * QD + VD, VD, W, 3);
        if (w == "mix.o") return mat(L.out, 0, W, VD, 0);
        if (w == "mix.norm") return L.dec_norm_weight && vec(L.onorm, VD);
    } else if (L.kind == MIX_LATENT) {
        const LatentParams & a = L.lat;
        const int64_t VD = (int64_t) a.heads * a.vdim;
        if (w == "mix.dq") return mat(L.lproj, 0, a.q_rank, W, 0);
        if (w == "mix.g") return mat(L.lproj, a.q_rank, VD, W, 1);
        if (w == "mix.dkv") return a.own_kv && mat(L.lproj, a.q_rank + VD, a.kv_rank + a.rot_dim, W, 2);
        if (w == "mix.dq.norm") return vec(L.dq_norm, a.q_rank);
        if (w == "mix.dkv.norm") return a.own_kv && vec(L.dkv_norm, a.kv_rank);
        if (w == "mix.uq") return mat(L.uq, 0, (int64_t) a.heads * (a.dim + a.rot_dim), a.q_rank, 0);
        if (w == "mix.uk") return mat(L.uk, 0, (int64_t) a.heads * a.dim, a.kv_rank, 0);
        if (w == "mix.uv") return mat(L.uv, 0, VD, a.kv_rank, 0);
        if (w == "mix.o") return mat(L.out, 0, W, VD, 0);
    }
    return false;
}

// ---------------------------------------------------------------------------------------------------------------
// Sapudra: configuration keys and tensor names.  Post-norm layers (layer norm with weight and bias on the sublayer's result, times
// residual_mult), a learned position table, windowed attention with grouped key / value heads and an RMS norm per query / key head, the
// squared-ReLU feed-forward, dense or "moe" (sigmoid router with a choice correction and expert groups, gated shared expert), soft-capped logits.
static int sapudra_configure(const Json & cfg, LayerList & ll, std::string & err) {
    ll.frame = FRAME_POSTNORM;
    ll.width = (int) cfg.integer("width", 0);
    ll.vocab = (int) cfg.integer("vocab", 0);
    ll.max_pos = (int) cfg.integer("max_positions", 0);
    ll.resid_mult = (float) cfg.number("residual_mult", 1.0);
    ll.logit_softcap = (float) cfg.number("logit_softcap", 0.0);
    ll.logit_scale = 1.f;
    if (const Json * nrm = cfg.get("norm")) ll.eps = (float) nrm->number("eps", 1e-6);
    const Json * layers = cfg.get("layers");
    if (ll.width <= 0 || ll.vocab <= 0 || ll.max_pos <= 0 || !layers || layers->kind != Json::ARR || layers->arr.empty()) { err = "width, vocab, max_positions and layers are required"; return PB200_EINVAL; }
    for (const Json & jl : layers->arr) {
        LLayer L;
        const std::string type = jl.string("type");
        const Json * mx = jl.get("mixer");
        if (!mx || mx->kind != Json::OBJ) { err = "layer without mixer"; return PB200_EINVAL; }
        if (type != "attention") { err = "unknown layer type '" + type + "'"; return PB200_ENOTSUP; }
        L.kind = MIX_ATTENTION;
        AttnParams & a = L.att;
        a.heads = (int) mx->integer("heads", 0);
        a.kv_heads = (int) mx->integer("kv_heads", a.heads);
        a.dim = (int) mx->integer("dim", 0);
        a.vdim = (int) mx->integer("vdim", a.dim);
        a.scale = (float) mx->number("scale", a.dim > 0 ? 1.0 / std::sqrt((double) a.dim) : 1.0);
        a.softcap = 0.f;
        a.gated = 0;
        a.window = 0;
        a.keep_first = 0;
        if (const Json * mk = mx->get("mask"))
            if (mk->kind == Json::OBJ) a.window = (int) std::min<long long>(mk->integer("size", 0), 1 << 30);
        L.qk_norm = true;
        if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.dim <= 0 || a.vdim <= 0 || a.vdim > 512) { err = "attention sizes"; return PB200_EINVAL; }
        const Json * mlp = jl.get("mlp");
        if (mlp && mlp->kind == Json::OBJ) {
            const std::string kind = mlp->string("kind", "dense");
            if (kind == "dense") {
                L.ff_kind = FF_RELU2;
                L.ff = (int) mlp->integer("ff", 0);
                if (L.ff <= 0) { err = "feed-forward size"; return PB200_EINVAL; }
            } else if (kind == "moe") {
                L.ff_kind = FF_MOE;
                L.route = ROUTE_SIGMOID_GROUPS;
                MoeParams & p = L.moe;
                p.act = 1;
                const Json * ex = mlp->get("expert"), * ro = mlp->get("router"), * sh = mlp->get("shared");
                if (!ex || ex->kind != Json::OBJ || !ro || ro->kind != Json::OBJ) { err = "moe needs expert and router"; return PB200_EINVAL; }
                p.ff = (int) ex->integer("ff", 0);
                L.ff = p.ff;
                p.experts = (int) ro->integer("experts", 0);
                p.top = (int) ro->integer("top", 0);
                p.route_scale = (float) ro->number("scale", 1.0);
                p.groups = p.keep_groups = 1;
                if (const Json * gr = ro->get("groups"))
                    if (gr->kind == Json::OBJ) { p.groups = (int) gr->integer("count", 1); p.keep_groups = (int) gr->integer("keep", p.groups); }
                if (p.ff <= 0 || p.experts <= 0 || p.top <= 0 || p.top > p.experts || p.top > 32 || p.experts > 4096 || p.groups <= 0 || p.experts % p.groups ||
                    p.keep_groups <= 0 || p.keep_groups > p.groups || (int64_t) p.keep_groups * (p.experts / p.groups) < p.top) { err = "router sizes"; return PB200_EINVAL; }
                if (sh && sh->kind == Json::OBJ) {
                    L.shared_ff = (int) sh->integer("ff", 0);
                    if (L.shared_ff <= 0) { err = "shared expert size"; return PB200_EINVAL; }
                }
            } else {
                err = "unknown feed-forward kind '" + kind + "'";
                return PB200_ENOTSUP;
            }
        }
        ll.layers.push_back(std::move(L));
    }
    for (int i = 0; i < (int) ll.layers.size(); i++) {
        LRun r;
        r.layer = i;
        ll.runs.push_back(r);
    }
    return 0;
}

static bool sapudra_resolve(LayerList & ll, const std::string & name, TensorPlace & o) {
    const int64_t W = ll.width;
    auto mat = [&](DenseW & m, int64_t row0, int64_t rows, int64_t cols, int part) { o.mat = &m; o.row0 = row0; o.rows = rows; o.cols = cols; o.part = part; return true; };
    auto vec = [&](VecF & v, int64_t n) { o.vec = &v; o.n = n; return true; };
    if (name == "embed") return mat(ll.embed, 0, ll.vocab, W, 0);
    if (name == "pos") return mat(ll.pos_table, 0, ll.max_pos, W, 0);
    if (name == "head") return mat(ll.head, 0, ll.vocab, W, 0);
    if (name == "final.norm") return vec(ll.final_norm, W);
    if (name == "final.norm.b") return vec(ll.final_norm_bias, W);
    int il = -1, used = 0;
    if (sscanf(name.c_str(), "l%d.%n", &il, &used) != 1 || used <= 0 || il < 0 || il >= (int) ll.layers.size()) return false;
    LLayer & L = ll.layers[(size_t) il];
    const std::string w = name.substr((size_t) used);
    if (w == "norm1") return vec(L.norm1, W);
    if (w == "norm1.b") return vec(L.norm1_bias, W);
    const AttnParams & a = L.att;
    const int64_t QD = (int64_t) a.heads * a.dim, KD = (int64_t) a.kv_heads * a.dim, VD = (int64_t) a.kv_heads * a.vdim;
    if (w == "mix.q") return mat(L.qkvg, 0, QD, W, 0);
    if (w == "mix.k") return mat(L.qkvg, QD, KD, W, 1);
    if (w == "mix.v") return mat(L.qkvg, QD + KD, VD, W, 2);
    if (w == "mix.q.norm") return vec(L.q_norm, a.dim);
    if (w == "mix.k.norm") return vec(L.k_norm, a.dim);
    if (w == "mix.o") return mat(L.out, 0, W, (int64_t) a.heads * a.vdim, 0);
    if (L.ff <= 0) return false;
    if (w == "norm2") return vec(L.norm2, W);
    if (w == "norm2.b") return vec(L.norm2_bias, W);
    if (w.compare(0, 4, "mlp.") != 0) return false;
    const std::string f = w.substr(4);
    if (L.ff_kind == FF_RELU2) {
        if (f == "up") return mat(L.gateup, 0, L.ff, W, 0);
        if (f == "down") return mat(L.down, 0, W, L.ff, 0);
        return false;
    }
    if (f == "router") { o.vec = &L.router; o.n = (int64_t) L.moe.experts * W; return true; }
    if (f == "correction") return vec(L.router_b, L.moe.experts);
    if (L.shared_ff > 0) {
        if (f == "shared.up") return mat(L.s_gateup, 0, L.shared_ff, W, 0);
        if (f == "shared.down") return mat(L.s_down, 0, W, L.shared_ff, 0);
        if (f == "shared.sg") return vec(L.shared_gate, W);
    }
    int e = -1, u2 = 0;
    if (sscanf(f.c_str(), "e%d.%n", &e, &u2) == 1 && u2 > 0 && e >= 0 && e < L.moe.experts) {
        const std::string leaf = f.substr((size_t) u2);
        if (leaf == "up") return mat(L.e_gateup, (int64_t) e * L.moe.ff, L.moe.ff, W, e);
        if (leaf == "down") return mat(L.e_down, (int64_t) e * W, W, L.moe.ff, e);
    }
    return false;
}

// ---------------------------------------------------------------------------------------------------------------
// Zevedra: configuration keys and tensor names.  The stream starts as embed[token] * scale + a hashed bigram row; every layer is
// x <- x + m mixer(norm x), x <- x + m ff(norm x) with an RMS norm of one learned number; a repeated block whose passes add the embedding
// output and a step vector.  Mixers are dual: "parallel" = windowed softmax attention (short convolution on q, k, v, interleaved partial
// rotation, unit RMS per head after it, values turned by their position, a gate per head) beside the gated delta rule, joined as
// a * left + b * right; "parallel_2" = causal attention with a sink (RMS norm with weight over the whole q / k projection before a
// rotate-half partial rotation, a gate per element) beside HGRN2, joined as the mean of the two normed results.  Feed-forward: SiLU-gated
// experts, sigmoid router, the plain scores of the chosen experts multiply their input.
static void plain_rotary_table(double base, int dims, std::vector<float> & freq) {
    freq.assign((size_t) std::max(dims / 2, 1), 0.f);
    for (int i = 0; i < dims / 2; i++) freq[(size_t) i] = (float) std::pow(base, -2.0 * i / dims);
}
static int zevedra_attention(const Json & jl, AttnParams & a, DualMix & d, LLayer & L, std::string & err) {
    a.heads = (int) jl.integer("heads", 0);
    a.kv_heads = (int) jl.integer("kv_heads", a.heads);
    a.dim = (int) jl.integer("dim", 0);
    a.vdim = (int) jl.integer("vdim", a.dim);
    a.scale = (float) jl.number("scale", a.dim > 0 ? 1.0 / std::sqrt((double) a.dim) : 1.0);
    a.softcap = 0.f;
    a.gated = 0;
    a.window = 0;
    a.keep_first = 0;
    if (const Json * mk = jl.get("mask"))
        if (mk->kind == Json::OBJ) a.window = (int) std::min<long long>(mk->integer("size", 0), 1 << 30);
    if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.dim <= 0 || a.vdim <= 0 || a.vdim > 512) { err = "attention sizes"; return PB200_EINVAL; }
    double base = 10000.0;
    d.rot_dims = 0;
    const Json * rot = jl.get("rot");
    if (rot && rot->kind == Json::OBJ) {
        base = rot->number("base", 10000.0);
        d.rot_dims = (int) rot->integer("dims", a.dim);
        if (d.rot_dims < 0 || d.rot_dims > a.dim || d.rot_dims % 2 || !(base > 0.0)) { err = "rotated dimensions"; return PB200_EINVAL; }
    }
    plain_rotary_table(base, d.rot_dims, L.rot_freq.preset);
    if (d.v_rot) {
        if (a.vdim % 2) { err = "rotated values need an even value size"; return PB200_EINVAL; }
        plain_rotary_table(base, a.vdim, L.vrot_freq.preset);
    }
    d.taps_l = (int) jl.integer("conv", 0);
    if (d.taps_l < 0 || d.taps_l > 64) { err = "convolution taps"; return PB200_EINVAL; }
    return 0;
}

static int zevedra_configure(const Json & cfg, LayerList & ll, std::string & err) {
    ll.frame = FRAME_PRERMS;
    ll.width = (int) cfg.integer("width", 0);
    ll.vocab = (int) cfg.integer("vocab", 0);
    ll.resid_mult = (float) cfg.number("residual_mult", 1.0);
    ll.logit_scale = 1.f;
    if (const Json * nrm = cfg.get("norm")) ll.eps = (float) nrm->number("eps", 1e-6);
    if (const Json * em = cfg.get("embedding")) {
        if (em->kind == Json::OBJ) {
            ll.embed_scale = (float) em->number("scale", 1.0);
            const Json * bg = em->get("bigram");
            if (bg && bg->kind == Json::OBJ) {
                ll.bigram.buckets = bg->integer("buckets", 0);
                ll.bigram.mul_prev = bg->integer("mul_prev", 0);
                ll.bigram.mul_cur = bg->integer("mul_cur", 0);
                if (ll.bigram.buckets <= 0 || ll.bigram.buckets > (1ll << 30)) { err = "bigram sizes"; return PB200_EINVAL; }
                // (a p + b c) mod n with the factors reduced first: the same row, and the products stay inside 64 bits for any factor
                ll.bigram.mul_prev = (ll.bigram.mul_prev % ll.bigram.buckets + ll.bigram.buckets) % ll.bigram.buckets;
                ll.bigram.mul_cur = (ll.bigram.mul_cur % ll.bigram.buckets + ll.bigram.buckets) % ll.bigram.buckets;
            }
        }
    }
    const Json * layers = cfg.get("layers");
    if (ll.width <= 0 || ll.vocab <= 0 || !layers || layers->kind != Json::ARR || layers->arr.empty()) { err = "width, vocab and layers are required"; return PB200_EINVAL; }
    for (const Json & jl : layers->arr) {
        LLayer L;
        L.kind = MIX_DUAL;
        DualMix & d = L.dual;
        const std::string type = jl.string("type");
        const Json * mx = jl.get("mixer");
        const Json * jle = mx && mx->kind == Json::OBJ ? mx->get("left") : nullptr, * jr = mx && mx->kind == Json::OBJ ? mx->get("right") : nullptr;
        if (!jle || jle->kind != Json::OBJ || !jr || jr->kind != Json::OBJ) { err = "a dual mixer needs left and right"; return PB200_EINVAL; }
        GatedLinParams & rp = d.rp;
        rp.heads = (int) jr->integer("heads", 0);
        rp.qk_heads = (int) jr->integer("kv_heads", rp.heads);
        rp.dim = (int) jr->integer("dim", 0);
        rp.vdim = (int) jr->integer("vdim", rp.dim);
        if (rp.heads <= 0 || rp.qk_heads <= 0 || rp.heads % rp.qk_heads || rp.dim <= 0 || rp.vdim <= 0 || rp.dim > 512) { err = "recurrence sizes"; return PB200_EINVAL; }
        AttnParams & a = L.att;
        if (type == "parallel") {
            d.rec = REC_DELTA; d.join = JOIN_SCALED_SUM;
            d.qk_norm = QKN_HEAD_UNIT; d.rot_layout = ROT_INTERLEAVED; d.v_rot = 1; d.gate_mode = 1;
            a.sink = 0;
            rp.delta = 1; rp.decay_per_channel = 0; rp.tied_key = 0;
            d.left_scale = (float) mx->number("left_scale", 1.0);
            d.right_scale = (float) mx->number("right_scale", 1.0);
            d.taps_r = (int) jr->integer("conv", 0);
        } else if (type == "parallel_2") {
            d.rec = REC_HGRN2; d.join = JOIN_NORMED_MEAN;
            d.qk_norm = QKN_WHOLE_WEIGHT; d.rot_layout = ROT_HALVES; d.v_rot = 0; d.gate_mode = 2;
            rp.delta = 0; rp.decay_per_channel = 1; rp.tied_key = 1;
            rp.qk_heads = rp.heads;
            d.left_scale = d.right_scale = 0.5f;
        } else {
            err = "unknown layer type '" + type + "'";
            return PB200_ENOTSUP;
        }
        int rc = zevedra_attention(*jle, a, d, L, err);
        if (rc) return rc;
        if (type == "parallel") {
            // every delta-rule input passes convolution + SiLU; a branch without taps is not part of the design
            if (d.taps_l < 1 || d.taps_r < 1 || d.taps_r > 64) { err = "parallel: convolution taps of both branches"; return PB200_EINVAL; }
            d.taps = std::max(d.taps_l, d.taps_r);
        } else {
            a.sink = 1;
            d.taps_l = d.taps_r = d.taps = 0;
        }
        // columns of the fused projection
        const int QD = a.heads * a.dim, KD = a.kv_heads * a.dim, VD = a.kv_heads * a.vdim, OD = a.heads * a.vdim;
        const int RQ = rp.qk_heads * rp.dim, RV = rp.heads * rp.vdim;
        int c = 0;
        d.c_q = c; c += QD;
        d.c_k = c; c += KD;
        d.c_v = c; c += VD;
        d.conv_l = c;
        if (d.rec == REC_DELTA) {
            d.c_rq = c; c += RQ;
            d.c_rk = c; c += RQ;
            d.c_rv = c; c += RV;
            d.conv_ch = c;
            d.c_g = c; c += a.heads;
            d.c_rb = c; c += rp.heads;
            d.c_ra = c; c += rp.heads;
            d.c_rg = c; c += RV;
        } else {
            d.conv_ch = 0;
            d.c_g = c; c += OD;
            d.c_rq = c; c += RQ;
            d.c_rk = c; c += RQ;     // forget-gate logits
            d.c_rv = c; c += RV;
        }
        d.cols = c;
        L.dconv_w.n_parts = d.taps > 0 ? 6 : 0;
        L.ff = 0;
        const Json * mlp = jl.get("mlp");
        if (mlp && mlp->kind == Json::OBJ) {
            const std::string kind = mlp->string("kind", "moe");
            if (kind != "moe") { err = "unknown feed-forward kind '" + kind + "'"; return PB200_ENOTSUP; }
            L.ff_kind = FF_MOE;
            L.route = ROUTE_SIGMOID_PLAIN;
            MoeParams & p = L.moe;
            p.act = 2;
            p.weight_on_input = 1;
            p.norm_weights = 0;
            p.route_scale = 1.f;
            p.groups = p.keep_groups = 1;
            const Json * ex = mlp->get("expert"), * ro = mlp->get("router");
            if (!ex || ex->kind != Json::OBJ || !ro || ro->kind != Json::OBJ) { err = "moe needs expert and router"; return PB200_EINVAL; }
            p.ff = (int) ex->integer("ff", 0);
            L.ff = p.ff;
            p.experts = (int) ro->integer("experts", 0);
            p.top = (int) ro->integer("top", 0);
            if (p.ff <= 0 || p.experts <= 0 || p.top <= 0 || p.top > p.experts || p.top > 32 || p.experts > 4096) { err = "router sizes"; return PB200_EINVAL; }
        }
        ll.layers.push_back(std::move(L));
    }
    const int nl = (int) ll.layers.size();
    ll.loop_times = 0;
    if (const Json * lp = cfg.get("loop")) {
        if (lp->kind == Json::OBJ) {
            ll.loop_start = (int) lp->integer("start", 0);
            ll.loop_stop = (int) lp->integer("stop", 0);
            ll.loop_times = (int) lp->integer("times", 1);
            if (ll.loop_start < 0 || ll.loop_stop > nl || ll.loop_start >= ll.loop_stop || ll.loop_times < 1) { err = "loop range"; return PB200_EINVAL; }
        }
    }
    for (int i = 0; i < nl;) {
        if (ll.loop_times > 0 && i == ll.loop_start) {
            for (int t = 0; t < ll.loop_times; t++)
                for (int k = ll.loop_start; k < ll.loop_stop; k++) {
                    LRun r;
                    r.layer = k;
                    r.pass = k == ll.loop_start ? t : -1;
                    ll.runs.push_back(r);
                }
            i = ll.loop_stop;
        } else {
            LRun r;
            r.layer = i++;
            ll.runs.push_back(r);
        }
    }
    return 0;
}

static bool zevedra_resolve(LayerList & ll, const std::string & name, TensorPlace & o) {
    const int64_t W = ll.width;
    auto mat = [&](DenseW & m, int64_t row0, int64_t rows, int64_t cols, int part) { o.mat = &m; o.row0 = row0; o.rows = rows; o.cols = cols; o.part = part; return true; };
    auto matc = [&](DenseW & m, int64_t col0, int64_t rows, int64_t cols, int part) { o.mat = &m; o.row0 = 0; o.col0 = col0; o.rows = rows; o.cols = cols; o.part = part; return true; };
    auto vec = [&](VecF & v, int64_t n) { o.vec = &v; o.n = n; return true; };
    // a tensor of n elements copied `times` times back to back: one number for a whole row, a weight that all heads share
    auto tiled = [&](VecF & v, int64_t n, int64_t times) { o.vec = &v; o.n = n; o.vrows = 1; o.vcols = n; o.vld = n; o.repeat = times; o.vrep = n; return true; };
    if (name == "embed") return mat(ll.embed, 0, ll.vocab, W, 0);
    if (name == "bigram") return ll.bigram.buckets > 0 && mat(ll.bigram_table, 0, ll.bigram.buckets + 1, W, 0);
    if (name == "head") return mat(ll.head, 0, ll.vocab, W, 0);
    if (name == "final.norm") return tiled(ll.final_norm, 1, W);
    if (name == "loop.step") return ll.loop_times > 0 && vec(ll.loop_step, (int64_t) ll.loop_times * W);
    int il = -1, used = 0;
    if (sscanf(name.c_str(), "l%d.%n", &il, &used) != 1 || used <= 0 || il < 0 || il >= (int) ll.layers.size()) return false;
    LLayer & L = ll.layers[(size_t) il];
    const std::string w = name.substr((size_t) used);
    if (w == "norm1") return tiled(L.norm1, 1, W);
    if (w.compare(0, 4, "mlp.") == 0 || w == "norm2") {
        if (L.ff <= 0) return false;
        if (w == "norm2") return tiled(L.norm2, 1, W);
        const std::string f = w.substr(4);
        if (f == "router") { o.vec = &L.router; o.n = (int64_t) L.moe.experts * W; return true; }
        int e = -1, u2 = 0;
        if (sscanf(f.c_str(), "e%d.%n", &e, &u2) == 1 && u2 > 0 && e >= 0 && e < L.moe.experts) {
            const std::string leaf = f.substr((size_t) u2);
            const int64_t ff = L.moe.ff;
            if (leaf == "gate") return mat(L.e_gateup, (int64_t) e * 2 * ff, ff, W, 2 * e);
            if (leaf == "up") return mat(L.e_gateup, (int64_t) e * 2 * ff + ff, ff, W, 2 * e + 1);
            if (leaf == "down") return mat(L.e_down, (int64_t) e * W, W, ff, e);
        }
        return false;
    }
    const DualMix & d = L.dual;
    const AttnParams & a = L.att;
    const GatedLinParams & rp = d.rp;
    const int64_t QD = (int64_t) a.heads * a.dim, KD = (int64_t) a.kv_heads * a.dim, VD = (int64_t) a.kv_heads * a.vdim, OD = (int64_t) a.heads * a.vdim;
    const int64_t RQ = (int64_t) rp.qk_heads * rp.dim, RV = (int64_t) rp.heads * rp.vdim;
    // a short convolution [channels][its taps] right-aligned in the layer's common tap count (the taps in front stay zero)
    auto conv = [&](int col0, int64_t ch, int taps, int part) {
        o.vec = &L.dconv_w; o.n = ch * taps; o.part = part;
        o.v0 = (int64_t) col0 * d.taps + (d.taps - taps); o.vrows = ch; o.vcols = taps; o.vld = d.taps; o.repeat = 1; o.vrep = 0;
        return true;
    };
    const bool sum = d.join == JOIN_SCALED_SUM;
    if (w.compare(0, 9, "mix.left.") == 0) {
        const std::string f = w.substr(9);
        if (f == "q") return mat(L.qkvg, d.c_q, QD, W, 0);
        if (f == "k") return mat(L.qkvg, d.c_k, KD, W, 1);
        if (f == "v") return mat(L.qkvg, d.c_v, VD, W, 2);
        if (f == "g") return mat(L.qkvg, d.c_g, d.gate_mode == 1 ? a.heads : OD, W, 3);
        if (f == "o") return sum ? matc(L.out, 0, W, OD, 0) : mat(L.out, 0, W, OD, 0);
        if (d.taps > 0) {
            if (f == "q.conv") return conv(d.c_q, QD, d.taps_l, 0);
            if (f == "k.conv") return conv(d.c_k, KD, d.taps_l, 1);
            if (f == "v.conv") return conv(d.c_v, VD, d.taps_l, 2);
        }
        if (d.qk_norm == QKN_WHOLE_WEIGHT) {
            if (f == "q.norm") return vec(L.q_norm, QD);
            if (f == "k.norm") return vec(L.k_norm, KD);
        }
        if (!sum && f == "out") return vec(L.join_wl, W);
        return false;
    }
    if (w.compare(0, 10, "mix.right.") == 0) {
        const std::string f = w.substr(10);
        if (f == "q") return mat(L.qkvg, d.c_rq, RQ, W, 4);
        if (f == "v") return mat(L.qkvg, d.c_rv, RV, W, 6);
        if (f == "norm") return tiled(L.onorm, rp.vdim, rp.heads);
        if (f == "o") return sum ? matc(L.out, OD, W, RV, 1) : mat(L.out_r, 0, W, RV, 0);
        if (d.rec == REC_DELTA) {
            if (f == "k") return mat(L.qkvg, d.c_rk, RQ, W, 5);
            if (f == "b") return mat(L.qkvg, d.c_rb, rp.heads, W, 7);
            if (f == "a") return mat(L.qkvg, d.c_ra, rp.heads, W, 8);
            if (f == "g") return mat(L.qkvg, d.c_rg, RV, W, 9);
            if (f == "A_log") return vec(L.A_log, rp.heads);
            if (f == "dt_bias") return vec(L.dt_bias, rp.heads);
            if (f == "q.conv") return conv(d.c_rq, RQ, d.taps_r, 3);
            if (f == "k.conv") return conv(d.c_rk, RQ, d.taps_r, 4);
            if (f == "v.conv") return conv(d.c_rv, RV, d.taps_r, 5);
        } else {
            if (f == "f") return mat(L.qkvg, d.c_rk, RQ, W, 5);
            if (f == "f.b") return vec(L.f_bias, RQ);
            if (f == "lower") return vec(L.f_lower, RQ);
            if (!sum && f == "out") return vec(L.join_wr, W);
        }
        return false;
    }
    return false;
}

static const ArchEntry g_archs[] = {
    {"llama", ARCH_KQUANT, 0, nullptr, nullptr},
    {"qwen2", ARCH_KQUANT, 2, nullptr, nullptr},
    {"Vamidra", ARCH_LAYERS, 0, vamidra_configure, vamidra_resolve},
    {"Mumizen", ARCH_LAYERS, 0, mumizen_configure, mumizen_resolve},
    {"Sapudra", ARCH_LAYERS, 0, sapudra_configure, sapudra_resolve},
    {"Zevedra", ARCH_LAYERS, 0, zevedra_configure, zevedra_resolve},
};
int arch_count() { return (int) (sizeof(g_archs) / sizeof(g_archs[0])); }
const ArchEntry * arch_at(int i) { return (i >= 0 && i < arch_count()) ? &g_archs[i] : nullptr; }
const ArchEntry * arch_find(const char * name) {
    if (!name) return nullptr;
    for (const ArchEntry & a : g_archs)
        if (strcmp(a.name, name) == 0) return &a;
    return nullptr;
}

// ---------------------------------------------------------------------------------------------------------------
static size_t esize(int type) { return type == T_BF16 ? 2 : 4; }

// every matrix / vector of the model with its size: allocation, completeness check, synthetic fill
template <typename FM, typename FV>
static void for_each_param(LayerList & ll, FM && fm, FV && fv) {
    const int64_t W = ll.width;
    fm(ll.embed, (int64_t) ll.vocab, W, 1);
    fm(ll.head, (int64_t) ll.vocab, W, 1);
    fv(ll.final_norm, W, 0);
    if (ll.frame == FRAME_POSTNORM) { fm(ll.pos_table, (int64_t) ll.max_pos, W, 1); fv(ll.final_norm_bias, W, 1); }
    if (ll.frame == FRAME_PRERMS && ll.bigram.buckets > 0) fm(ll.bigram_table, ll.bigram.buckets + 1, W, 1);
    if (ll.loop_times > 0) {
        if (ll.frame != FRAME_PRERMS) fm(ll.loop_in, W, 2 * W, 1);
        fv(ll.loop_step, (int64_t) ll.loop_times * W, 1);
    }
    int il = 0;
    for (LLayer & L : ll.layers) {
        fv(L.norm1, W, 0);
        if (ll.frame == FRAME_SANDWICH) fv(L.norm1b, W, 0);
        else if (ll.frame == FRAME_POSTNORM) fv(L.norm1_bias, W, 1);
        else if (ll.frame == FRAME_PRENORM) { fv(L.shift, W, 5); fv(L.dwa, il + 2, 6); }
        il++;
        if (L.kind == MIX_ATTENTION) {
            fm(L.qkvg, attn_qkvg_cols(L.att), W, L.att.gated ? 4 : 3);
            if (L.qk_norm) { fv(L.q_norm, L.att.dim, 0); fv(L.k_norm, L.att.dim, 0); }
            fm(L.out, W, (int64_t) L.att.heads * L.att.vdim, 1);
        } else if (L.kind == MIX_MAMBA2) {
            const Mamba2Params & p = L.ssm;
            fm(L.in, mamba2_in_cols(p), W, 1);
            fv(L.conv_w, (int64_t) mamba2_conv_channels(p) * p.conv, 2); fv(L.conv_b, mamba2_conv_channels(p), 1);
            fv(L.dt_bias, p.heads, 3); fv(L.A_log, p.heads, 4); fv(L.D, p.heads, 0); fv(L.gnorm, mamba2_inner(p), 0);
            fm(L.out, W, mamba2_inner(p), 1);
        } else if (L.kind == MIX_DECAY) {
            const int64_t QD = (int64_t) L.dec.heads * L.dec.dim, VD = (int64_t) L.dec.heads * L.dec.vdim;
            fm(L.qkvg, 2 * QD + 2 * VD, W, 4);
            fm(L.out, W, VD, 1);
            fv(L.decay, L.dec.heads, 0);
            if (L.dec_norm_weight) fv(L.onorm, VD, 0);
        } else if (L.kind == MIX_DUAL) {
            const DualMix & d = L.dual;
            const AttnParams & a = L.att;
            const int64_t OD = (int64_t) a.heads * a.vdim, RQ = (int64_t) d.rp.qk_heads * d.rp.dim, RV = (int64_t) d.rp.heads * d.rp.vdim;
            fm(L.qkvg, d.cols, W, d.rec == REC_DELTA ? 10 : 7);
            fv(L.rot_freq, (int64_t) L.rot_freq.preset.size(), 0);
            if (d.v_rot) fv(L.vrot_freq, (int64_t) L.vrot_freq.preset.size(), 0);
            if (d.taps > 0) fv(L.dconv_w, (int64_t) d.conv_ch * d.taps, 2);
            if (d.qk_norm == QKN_WHOLE_WEIGHT) { fv(L.q_norm, (int64_t) a.heads * a.dim, 0); fv(L.k_norm, (int64_t) a.kv_heads * a.dim, 0); }
            fv(L.onorm, RV, 0);
            if (d.rec == REC_DELTA) { fv(L.A_log, d.rp.heads, 4); fv(L.dt_bias, d.rp.heads, 3); }
            else { fv(L.f_bias, RQ, 1); fv(L.f_lower, RQ, 5); }
            if (d.join == JOIN_SCALED_SUM) {
                fm(L.out, W, OD + RV, 2);
            } else {
                fm(L.out, W, OD, 1); fm(L.out_r, W, RV, 1);
                fv(L.join_wl, W, 0); fv(L.join_wr, W, 0);
            }
        } else {
            const LatentParams & a = L.lat;
            fm(L.lproj, latent_proj_cols(a), W, a.own_kv ? 3 : 2);
            fv(L.dq_norm, a.q_rank, 0);
            if (a.own_kv) fv(L.dkv_norm, a.kv_rank, 0);
            fv(L.rot_freq, (int64_t) L.rot_freq.preset.size(), 0);
            fm(L.uq, (int64_t) a.heads * (a.dim + a.rot_dim), a.q_rank, 1);
            fm(L.uk, (int64_t) a.heads * a.dim, a.kv_rank, 1);
            fm(L.uv, (int64_t) a.heads * a.vdim, a.kv_rank, 1);
            fm(L.out, W, (int64_t) a.heads * a.vdim, 1);
        }
        if (L.ff > 0) {
            fv(L.norm2, W, 0);
            if (ll.frame == FRAME_SANDWICH) fv(L.norm2b, W, 0);
            if (ll.frame == FRAME_POSTNORM) fv(L.norm2_bias, W, 1);
            if (L.ff_kind == FF_MOE) {
                const int gated = L.moe.act == 1 ? 1 : 2;   // rows per expert: up only, or gate | up
                fm(L.e_gateup, (int64_t) L.moe.experts * moe_up_rows(L.moe), W, gated * L.moe.experts);
                fm(L.e_down, (int64_t) L.moe.experts * W, L.moe.ff, L.moe.experts);
                fv(L.router, (int64_t) L.moe.experts * W, 7);
                if (L.route != ROUTE_SIGMOID_PLAIN) fv(L.router_b, L.moe.experts, 1);
                if (L.shared_ff > 0) {
                    fm(L.s_gateup, gated * (int64_t) L.shared_ff, W, gated); fm(L.s_down, W, L.shared_ff, 1);
                    if (L.route == ROUTE_SIGMOID_GROUPS) fv(L.shared_gate, W, 7);
                }
            } else if (L.ff_kind == FF_RELU2) {
                fm(L.gateup, (int64_t) L.ff, W, 1);
                fm(L.down, W, L.ff, 1);
            } else {
                fm(L.gateup, 2 * (int64_t) L.ff, W, 2);
                fm(L.down, W, L.ff, 1);
            }
        }
    }
}

static int ll_alloc_params(pb200_model * m) {
    LayerList & ll = *m->ll;
    int rc = 0;
    int64_t bytes = 0;
    for_each_param(
        ll,
        [&](DenseW & d, int64_t N, int64_t K, int parts) {
            if (rc) return;
            d.N = N; d.K = K; d.filled.assign((size_t) parts, 0);
            const size_t b = (size_t) N * K * esize(ll.ctype);
            rc = m->alloc(&d.data, b + 16);
            bytes += (int64_t) b;
        },
        [&](VecF & v, int64_t n, int) {
            if (rc) return;
            v.n = n; v.filled = false;
            v.parts.assign((size_t) std::max(v.n_parts, 0), 0);
            rc = m->alloc((void **) &v.data, (size_t) n * 4);
            if (!rc) rc = (int) cudaMemset(v.data, 0, (size_t) n * 4);   // entries no tensor fills (padding taps) are zero
            bytes += n * 4;
            if (!rc && !v.preset.empty()) {   // fixed by the configuration
                rc = (int) cudaMemcpy(v.data, v.preset.data(), (size_t) n * 4, cudaMemcpyHostToDevice);
                v.filled = true;
            }
        });
    ll.weight_bytes = bytes;
    return rc;
}

static void bf16_to_f32(const uint16_t * s, float * d, size_t n) {
    for (size_t i = 0; i < n; i++) { const uint32_t b = (uint32_t) s[i] << 16; memcpy(d + i, &b, 4); }
}
static void f32_to_bf16(const float * s, uint16_t * d, size_t n) {   // round to nearest even
    for (size_t i = 0; i < n; i++) {
        uint32_t b;
        memcpy(&b, s + i, 4);
        if ((b & 0x7fffffffu) > 0x7f800000u) { d[i] = (uint16_t) ((b >> 16) | 0x40); continue; }
        b += 0x7fffu + ((b >> 16) & 1u);
        d[i] = (uint16_t) (b >> 16);
    }
}

}  // namespace pb

using namespace pb;

// ---------------------------------------------------------------------------------------------------------------
// entry points used by engine.cu's dispatch (the public ABI functions of the model object forward here when m->ll is set)
int ll_set_tensor(pb200_model * m, const char * name, int type, const void * host, size_t nbytes) {
    LayerList & ll = *m->ll;
    if (m->finalized) return PB200_ESTATE;
    if (type != T_F32 && type != T_BF16) return PB200_ENOTSUP;
    TensorPlace pl;
    if (!ll.arch->resolve(ll, name, pl)) return PB200_EINVAL;
    const int64_t count = pl.mat ? pl.rows * pl.cols : pl.n;
    if (nbytes != (size_t) count * esize(type)) return PB200_EINVAL;
    cudaSetDevice(m->device);
    const int dtype = pl.mat ? ll.ctype : T_F32;
    std::vector<uint8_t> conv;
    const void * src = host;
    if (type != dtype) {
        conv.resize((size_t) count * esize(dtype));
        if (dtype == T_F32) bf16_to_f32((const uint16_t *) host, (float *) conv.data(), (size_t) count);
        else f32_to_bf16((const float *) host, (uint16_t *) conv.data(), (size_t) count);
        src = conv.data();
    }
    if (pl.mat) {
        const size_t es = esize(dtype);
        if (pl.col0 < 0 || pl.col0 + pl.cols > pl.mat->K || pl.row0 + pl.rows > pl.mat->N || (size_t) pl.part >= pl.mat->filled.size()) return PB200_EINVAL;
        CK(cudaMemcpy2D((uint8_t *) pl.mat->data + ((size_t) pl.row0 * pl.mat->K + (size_t) pl.col0) * es, (size_t) pl.mat->K * es, src, (size_t) pl.cols * es,
                        (size_t) pl.cols * es, (size_t) pl.rows, cudaMemcpyHostToDevice));
        pl.mat->filled[(size_t) pl.part] = 1;
    } else if (pl.vrows > 0) {
        if (pl.vrows * pl.vcols != pl.n || pl.vcols > pl.vld || pl.repeat < 1) return PB200_EINVAL;
        for (int64_t r = 0; r < pl.repeat; r++) {
            const int64_t first = pl.v0 + r * pl.vrep;
            if (first < 0 || first + (pl.vrows - 1) * pl.vld + pl.vcols > pl.vec->n) return PB200_EINVAL;
            CK(cudaMemcpy2D(pl.vec->data + first, (size_t) pl.vld * 4, src, (size_t) pl.vcols * 4, (size_t) pl.vcols * 4, (size_t) pl.vrows, cudaMemcpyHostToDevice));
        }
        if (pl.vec->parts.empty()) pl.vec->filled = true;
        else if ((size_t) pl.part < pl.vec->parts.size()) pl.vec->parts[(size_t) pl.part] = 1;
        else return PB200_EINVAL;
    } else {
        if (pl.n != pl.vec->n) return PB200_EINVAL;
        CK(cudaMemcpy(pl.vec->data, src, (size_t) count * 4, cudaMemcpyHostToDevice));
        pl.vec->filled = true;
    }
    return 0;
}

namespace {
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
template <typename OT>
__global__ void k_fill_uniform(OT * p, int64_t n, float base, float half_range, uint64_t seed) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float u = (float) (mix64(seed + (uint64_t) i * 0x9E3779B97F4A7C15ull) >> 40) * (1.0f / 16777216.0f);
    const float v = base + half_range * (2.f * u - 1.f);
    if constexpr (sizeof(OT) == 2) p[i] = __float2bfloat16_rn(v); else p[i] = v;
}
}  // namespace

// random weights generated on the device (benchmarks without a checkpoint): matrices uniform with standard deviation ~ 1/sqrt(K)
int ll_synth(pb200_model * m, uint64_t seed) {
    LayerList & ll = *m->ll;
    if (m->finalized) return PB200_ESTATE;
    cudaSetDevice(m->device);
    uint64_t sd = seed * 0x100000001B3ull + 17;
    int rc = 0;
    for_each_param(
        ll,
        [&](DenseW & d, int64_t N, int64_t K, int) {
            if (rc) return;
            const int64_t n = N * K;
            const float hr = 1.7320508f / sqrtf((float) K);
            if (ll.ctype == T_BF16) k_fill_uniform<__nv_bfloat16><<<(unsigned) ((n + 255) / 256), 256, 0, m->stream>>>((__nv_bfloat16 *) d.data, n, 0.f, hr, ++sd);
            else k_fill_uniform<float><<<(unsigned) ((n + 255) / 256), 256, 0, m->stream>>>((float *) d.data, n, 0.f, hr, ++sd);
            rc = (int) cudaGetLastError();
            std::fill(d.filled.begin(), d.filled.end(), 1);
        },
        [&](VecF & v, int64_t n, int kind) {   // kind 0: around one, 1: around zero, 2: convolution taps, 3: dt bias, 4: log of the decay rate,
            if (rc || !v.preset.empty()) return;   // 5: shift blend in [0, 1], 6: depth-average weights around 1 / n, 7: router rows
            const float base = kind == 0 ? 1.f : kind == 3 ? -2.f : kind == 4 ? 0.5f : kind == 5 ? 0.5f : kind == 6 ? 1.f / (float) n : 0.f;
            const float hr = kind == 0 ? 0.05f : kind == 1 ? 0.02f : kind == 2 ? 0.5f : kind == 5 ? 0.5f : kind == 6 ? 0.5f / (float) n
                             : kind == 7 ? 1.7320508f / sqrtf((float) ll.width) : 1.f;
            k_fill_uniform<float><<<(unsigned) ((n + 255) / 256), 256, 0, m->stream>>>(v.data, n, base, hr, ++sd);
            rc = (int) cudaGetLastError();
            v.filled = true;
            std::fill(v.parts.begin(), v.parts.end(), 1);
        });
    if (rc) return rc;
    return (int) cudaStreamSynchronize(m->stream);
}

int ll_finalize(pb200_model * m) {
    LayerList & ll = *m->ll;
    if (m->finalized) return 0;
    cudaSetDevice(m->device);
    bool complete = true;
    for_each_param(
        ll, [&](DenseW & d, int64_t, int64_t, int) { for (uint8_t f : d.filled) complete = complete && f; },
        [&](VecF & v, int64_t, int) {
            if (v.parts.empty()) complete = complete && v.filled;
            else for (uint8_t f : v.parts) complete = complete && f;
        });
    if (!complete) return PB200_ESTATE;
    // state arena layout of one slot
    int64_t off = 0;
    ll.ctx_limited = false;
    for (LRun & r : ll.runs) {
        LLayer & L = ll.layers[(size_t) r.layer];
        if (ll.frame == FRAME_PRENORM) { r.shift_off = off; off += ll.width; off = (off + 3) / 4 * 4; }
        r.state_off = off;
        if (L.kind == MIX_DECAY) {
            off += (int64_t) L.dec.heads * L.dec.dim * L.dec.vdim;
        } else if (L.kind == MIX_LATENT) {
            L.lat.cache_rows = ll.n_ctx;
            ll.ctx_limited = true;
            if (L.lat.own_kv) off += (int64_t) ll.n_ctx * latent_row(L.lat);
            else r.state_off = ll.runs[(size_t) L.kv_from].state_off;   // FRAME_PRENORM: run i is layer i
        } else if (L.kind == MIX_ATTENTION || L.kind == MIX_DUAL) {
            L.att.cache_rows = attn_cache_rows(L.att.window, L.att.keep_first, ll.n_ctx);
            if (L.att.cache_rows >= ll.n_ctx) ll.ctx_limited = true;
            off += (int64_t) L.att.cache_rows * L.att.kv_heads * (L.att.dim + L.att.vdim);
            if (L.kind == MIX_DUAL) {   // then the convolution's last inputs and the recurrence's state
                const DualMix & d = L.dual;
                off = (off + 3) / 4 * 4;
                off += (int64_t) std::max(d.taps - 1, 0) * d.conv_ch;
                off = (off + 3) / 4 * 4;
                off += (int64_t) d.rp.heads * d.rp.dim * d.rp.vdim;
            }
        } else {
            off += (int64_t) (L.ssm.conv - 1) * mamba2_conv_channels(L.ssm) + (int64_t) L.ssm.heads * L.ssm.state * L.ssm.vdim;
        }
        off = (off + 3) / 4 * 4;
    }
    ll.slot_floats = std::max<int64_t>(off, 4);
    if (ll.n_seq <= 0) {   // as many slots as 8 GiB of state (or an eighth of the free device memory, if that is more) hold, between 4 and 256
        size_t mem_free = 0, mem_total = 0;
        if (cudaMemGetInfo(&mem_free, &mem_total) != cudaSuccess) mem_free = 0;
        const int64_t fit = std::max<int64_t>(8ll << 30, (int64_t) (mem_free / 8)) / (ll.slot_floats * 4);
        ll.n_seq = (int) std::min<int64_t>(256, std::max<int64_t>(4, fit));
    }
    CK(m->alloc((void **) &ll.state, (size_t) ll.slot_floats * 4 * (size_t) ll.n_seq));
    CK(cudaMemset(ll.state, 0, (size_t) ll.slot_floats * 4 * (size_t) ll.n_seq));
    ll.seq_len.assign((size_t) ll.n_seq, -1);
    ll.seq_prev.assign((size_t) ll.n_seq, -1);
    m->n_seq = ll.n_seq;
    m->weight_bytes = ll.weight_bytes;
    m->finalized = true;
    return 0;
}

static void ll_drop_graphs(LayerList & ll);
void ll_free(pb200_model * m) {
    LayerList * ll = m->ll;
    if (!ll) return;
    ll_drop_graphs(*ll);
    for (void * p : ll->scratch) cudaFree(p);
    if (ll->meta_dev) cudaFree(ll->meta_dev);
    if (ll->meta_host) cudaFreeHost(ll->meta_host);
    if (ll->greedy_host) cudaFreeHost(ll->greedy_host);
    if (ll->logits_host) cudaFreeHost(ll->logits_host);
    if (ll->moe_count_host) cudaFreeHost(ll->moe_count_host);
    if (ll->lat_part) cudaFree(ll->lat_part);
    if (ll->tap) cudaFree(ll->tap);
    for (cudaEvent_t e : ll->prof_ev) cudaEventDestroy(e);
    if (ll->ev_fork) cudaEventDestroy(ll->ev_fork);
    if (ll->ev_join) cudaEventDestroy(ll->ev_join);
    if (ll->side) cudaStreamDestroy(ll->side);
    delete ll;
    m->ll = nullptr;
}

// ---- sequence slots ----
int ll_seq_alloc(pb200_model * m) {
    LayerList & ll = *m->ll;
    if (!m->finalized) return PB200_ESTATE;
    for (int s = 0; s < ll.n_seq; s++)
        if (ll.seq_len[(size_t) s] < 0) {
            cudaSetDevice(m->device);
            // a slot that is handed out again starts from the empty state: zero convolution inputs, zero recurrent state, no cached keys
            if (cudaMemsetAsync(ll.state + (int64_t) s * ll.slot_floats, 0, (size_t) ll.slot_floats * 4, m->stream) != cudaSuccess) return PB200_ENOMEM;
            ll.seq_len[(size_t) s] = 0;
            ll.seq_prev[(size_t) s] = -1;
            return s;
        }
    return PB200_ENOMEM;
}
int ll_seq_free(pb200_model * m, int slot) {
    LayerList & ll = *m->ll;
    if (slot < 0 || slot >= ll.n_seq || ll.seq_len[(size_t) slot] < 0) return PB200_EINVAL;
    ll.seq_len[(size_t) slot] = -1;
    return 0;
}
int ll_seq_length(pb200_model * m, int slot) {
    LayerList & ll = *m->ll;
    if (slot < 0 || slot >= ll.n_seq) return PB200_EINVAL;
    return ll.seq_len[(size_t) slot];
}

// ---- scratch ----
static void ll_drop_graphs(LayerList & ll) {
    for (auto & kv : ll.graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    ll.graphs.clear();
}
static int ll_reserve(pb200_model * m, int T, int nW, int nE) {
    LayerList & ll = *m->ll;
    const bool grow = T > ll.capT || nW > ll.capW || (size_t) 2 * T + 4 * (size_t) nE + 1 + (size_t) nW + 64 > ll.meta_cap;
    if (grow) ll_drop_graphs(ll);   // captured steps hold the addresses of buffers that are about to move
    if (T > ll.capT || nW > ll.capW) {
        CK(cudaStreamSynchronize(m->stream));
        for (void * p : ll.scratch) cudaFree(p);
        ll.scratch.clear();
        const int cT = std::max(T, ll.capT), cW = std::max(nW, ll.capW);
        ll.capT = ll.capW = 0;
        int64_t maxact = ll.width, maxact2 = ll.width, maxbig = ll.width, maxch = 1, maxinner = 1, maxb2 = 0, maxb3 = 0, maxb4 = 0, maxkr = 0;
        int64_t moe_top = 0, moe_topff = 0, moe_e = 0;
        for (const LLayer & L : ll.layers) {
            if (L.kind == MIX_ATTENTION) {
                maxact = std::max<int64_t>(maxact, (int64_t) L.att.heads * L.att.vdim);
                maxbig = std::max<int64_t>(maxbig, attn_qkvg_cols(L.att));
            } else if (L.kind == MIX_MAMBA2) {
                maxact = std::max<int64_t>(maxact, mamba2_inner(L.ssm));
                maxbig = std::max<int64_t>(maxbig, mamba2_in_cols(L.ssm));
                maxch = std::max<int64_t>(maxch, mamba2_conv_channels(L.ssm));
                maxinner = std::max<int64_t>(maxinner, mamba2_inner(L.ssm));
            } else if (L.kind == MIX_DECAY) {
                const int64_t QD = (int64_t) L.dec.heads * L.dec.dim, VD = (int64_t) L.dec.heads * L.dec.vdim;
                maxact = std::max(maxact, VD);
                maxbig = std::max(maxbig, 2 * QD + 2 * VD);
                maxinner = std::max(maxinner, VD);
            } else if (L.kind == MIX_DUAL) {
                const DualMix & d = L.dual;
                const int64_t OD = (int64_t) L.att.heads * L.att.vdim, RV = (int64_t) d.rp.heads * d.rp.vdim;
                maxact = std::max(maxact, OD + RV);
                maxact2 = std::max(maxact2, RV);
                maxbig = std::max<int64_t>(maxbig, d.cols);
                maxch = std::max<int64_t>(maxch, d.conv_ch);
                maxinner = std::max(maxinner, RV);
                maxb2 = std::max(maxb2, OD);                       // the attention result before it is turned back
                maxb4 = std::max<int64_t>(maxb4, 2 * ll.width);    // the two branch results before they are normed and joined
            } else {
                const LatentParams & a = L.lat;
                const int64_t H = a.heads;
                maxact = std::max(maxact, H * a.vdim);
                maxact2 = std::max<int64_t>(maxact2, std::max(a.q_rank, a.kv_rank));
                maxbig = std::max<int64_t>(maxbig, latent_proj_cols(a));
                maxb2 = std::max(maxb2, H * (a.dim + a.rot_dim));
                maxb3 = std::max(maxb3, std::max(H * a.dim, H * latent_row(a)));
                maxb4 = std::max(maxb4, std::max(H * a.vdim, H * a.kv_rank));
                maxkr = std::max<int64_t>(maxkr, a.rot_dim);
            }
            if (L.ff_kind == FF_MOE && L.ff > 0) {
                maxact2 = std::max<int64_t>(maxact2, L.shared_ff);
                maxbig = std::max<int64_t>(maxbig, 2 * (int64_t) L.shared_ff);
                moe_top = std::max<int64_t>(moe_top, L.moe.top);
                moe_topff = std::max<int64_t>(moe_topff, (int64_t) L.moe.top * L.moe.ff);
                moe_e = std::max<int64_t>(moe_e, L.moe.experts);
            } else {
                maxact = std::max<int64_t>(maxact, L.ff);
                maxact2 = std::max<int64_t>(maxact2, L.ff);
                maxbig = std::max<int64_t>(maxbig, 2 * (int64_t) L.ff);
            }
        }
        auto grab = [&](void ** p, size_t bytes) -> int {
            cudaError_t e = cudaMalloc(p, (bytes + 255) / 256 * 256 + 256);
            if (e != cudaSuccess) return (int) e;
            ll.scratch.push_back(*p);
            return 0;
        };
        const size_t W = (size_t) ll.width, t = (size_t) cT, es = esize(ll.ctype);
        CK(grab((void **) &ll.x, t * W * 4)); CK(grab((void **) &ll.x0, t * W * 4)); CK(grab((void **) &ll.xalt, t * W * 4));
        CK(grab((void **) &ll.msub, t * W * 4));
        CK(grab((void **) &ll.big, t * (size_t) maxbig * 4));
        CK(grab((void **) &ll.xbc, t * (size_t) maxch * 4));
        CK(grab((void **) &ll.yssm, t * (size_t) maxinner * 4));
        CK(grab(&ll.act, t * (size_t) maxact * es));
        CK(grab(&ll.act2, t * (size_t) maxact2 * es));
        if (ll.frame == FRAME_PRENORM) CK(grab((void **) &ll.hist, (ll.layers.size() + 1) * t * W * 4));
        if (maxb2) CK(grab((void **) &ll.big2, t * (size_t) maxb2 * 4));
        if (maxb3) CK(grab((void **) &ll.big3, t * (size_t) maxb3 * 4));
        if (maxb4) CK(grab((void **) &ll.big4, t * (size_t) maxb4 * 4));
        if (maxkr || maxb3) CK(grab((void **) &ll.krb, t * (size_t) std::max<int64_t>(maxkr, 1) * 4));
        if (moe_top) {
            const size_t pairs = t * (size_t) moe_top;
            CK(grab((void **) &ll.moe_idx, pairs * 4)); CK(grab((void **) &ll.moe_wt, pairs * 4)); CK(grab((void **) &ll.moe_sg, t * 4));
            CK(grab((void **) &ll.moe_perm, pairs * 4)); CK(grab((void **) &ll.moe_row_of, pairs * 4));
            CK(grab((void **) &ll.moe_count, (size_t) moe_e * 4)); CK(grab((void **) &ll.moe_start, (size_t) moe_e * 4));
            CK(grab(&ll.moe_y, t * (size_t) moe_topff * es)); CK(grab(&ll.moe_hs, pairs * W * es));
            CK(grab((void **) &ll.moe_gu, t * (size_t) moe_topff * 2 * 4)); CK(grab((void **) &ll.moe_ds, pairs * W * 4));
            if (!ll.moe_count_host) CK(cudaMallocHost((void **) &ll.moe_count_host, (size_t) 2 * 4096 * 4));
        }
        CK(grab(&ll.actw, (size_t) cW * W * es));
        CK(grab((void **) &ll.logits, (size_t) cW * (size_t) ll.vocab * 4));
        CK(grab((void **) &ll.greedy_dev, (size_t) cW * 4));
        if (ll.greedy_host) cudaFreeHost(ll.greedy_host);
        ll.greedy_host = nullptr;
        CK(cudaMallocHost((void **) &ll.greedy_host, (size_t) cW * 4));
        ll.capT = cT; ll.capW = cW;
    }
    size_t need_part = 0;
    for (const LLayer & L : ll.layers)
        if (L.kind == MIX_LATENT)
            need_part = std::max(need_part, (size_t) nE * (size_t) latent_decode_splits(ll.n_ctx) * (size_t) L.lat.heads * (size_t) (L.lat.kv_rank + 2));
        else if (L.kind == MIX_ATTENTION || L.kind == MIX_DUAL)
            need_part = std::max(need_part, attn_decode_part_floats(L.att, nE));
    if (need_part > ll.lat_part_cap) {
        CK(cudaStreamSynchronize(m->stream));
        ll_drop_graphs(ll);
        if (ll.lat_part) cudaFree(ll.lat_part);
        ll.lat_part = nullptr; ll.lat_part_cap = 0;
        CK(cudaMalloc((void **) &ll.lat_part, need_part * 2 * 4));
        ll.lat_part_cap = need_part * 2;
    }
    const size_t need_meta = (size_t) 2 * T + 4 * (size_t) nE + 1 + (size_t) nW + 64;
    if (need_meta > ll.meta_cap) {
        CK(cudaStreamSynchronize(m->stream));
        if (ll.meta_dev) cudaFree(ll.meta_dev);
        if (ll.meta_host) cudaFreeHost(ll.meta_host);
        ll.meta_dev = nullptr; ll.meta_host = nullptr; ll.meta_cap = 0;
        const size_t cap = need_meta * 2;
        CK(cudaMalloc((void **) &ll.meta_dev, cap * 4));
        CK(cudaMallocHost((void **) &ll.meta_host, cap * 4));
        ll.meta_cap = cap;
    }
    const size_t need_lh = (size_t) std::max(nW, 1) * (size_t) ll.vocab;
    if (need_lh > ll.logits_host_cap) {
        CK(cudaStreamSynchronize(m->stream));
        if (ll.logits_host) cudaFreeHost(ll.logits_host);
        ll.logits_host = nullptr; ll.logits_host_cap = 0;
        CK(cudaMallocHost((void **) &ll.logits_host, need_lh * 4));
        ll.logits_host_cap = need_lh;
    }
    return 0;
}

// One homogeneous ragged batch through every layer run.  `prefill`: every entry starts at position 0 (keys and values are read from
// the batch); otherwise every entry brings one token (keys and values come from the slot's cache).  Rows `want_dev[0..nW)` (token
// indices of the batch) go through the final norm and the output head into logits rows lrow0 ...
enum : int { CAT_DENSE = 0, CAT_ATTN = 1, CAT_CONV = 2, CAT_SCAN = 3, CAT_NORM = 4, CAT_ELEM = 5, CAT_HEAD = 6, CAT_TOTAL = 7, CAT_MOE = 8, CAT_LATENT = 9 };
static int prof_mark(pb200_model * m, int cat) {   // an event before the launch of a category; the next mark (or the end) closes its interval
    LayerList & ll = *m->ll;
    if (!ll.prof_on) return 0;
    const size_t i = ll.prof_cat.size();
    if (ll.prof_ev.size() <= i) { cudaEvent_t e; CK(cudaEventCreate(&e)); ll.prof_ev.push_back(e); }
    ll.prof_cat.push_back(cat);
    return (int) cudaEventRecord(ll.prof_ev[i], m->stream);
}
#define CAT(c) CK(prof_mark(m, c))

static int tap_prepare(pb200_model * m, int T) {
    LayerList & ll = *m->ll;
    if (!ll.tap_on) return 0;
    const int64_t need = (int64_t) ll.runs.size() * T * ll.width;
    if (need > ll.tap_cap) {
        CK(cudaStreamSynchronize(m->stream));
        if (ll.tap) cudaFree(ll.tap);
        ll.tap = nullptr; ll.tap_cap = 0;
        CK(cudaMalloc((void **) &ll.tap, (size_t) need * 4));
        ll.tap_cap = need;
    }
    ll.tap_floats = need;
    ll.tap_T = T;
    return 0;
}

// ---- mixers: out[t] = (resid ? resid[t] : 0) + mixer(ll.act[t]); ll.act holds the mixer's input in the operand type ----
static int mix_attention(pb200_model * m, const BatchView & b, bool prefill, const LRun & r, LLayer & L, const float * resid, float * out) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    const AttnParams & a = L.att;
    const int C = attn_qkvg_cols(a);
    float * sbase = ll.state + r.state_off;
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, W, L.qkvg.data, W, ll.big, C, T, C, W, nullptr, nullptr, 0, 1.f, st));
    float * kc = sbase, * vc = sbase + (int64_t) a.cache_rows * a.kv_heads * a.dim;
    CAT(CAT_ATTN);
    if (L.qk_norm) CK(launch_attn_qknorm_kv_store(ll.big, b, a, L.q_norm.data, L.k_norm.data, ll.eps, kc, vc, ll.slot_floats, st));
    else CK(launch_attn_kv_store(ll.big, b, a, kc, vc, ll.slot_floats, st));
    if (prefill) CK(launch_attn_window_prefill(ll.big, b, a, ll.act, ct, st));
    else CK(launch_attn_window_decode(ll.big, b, a, kc, vc, ll.slot_floats, ll.act, ct, st, ll.lat_part));
    CAT(CAT_DENSE);
    return launch_dense(ct, ll.act, (int64_t) a.heads * a.vdim, L.out.data, (int64_t) a.heads * a.vdim, out, W, T, W, a.heads * a.vdim, nullptr, resid, W, 1.f, st);
}
static int mix_mamba2(pb200_model * m, const BatchView & b, const LRun & r, LLayer & L, const float * resid, float * out) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    const Mamba2Params & p = L.ssm;
    const int U = mamba2_in_cols(p), inner = mamba2_inner(p);
    float * sbase = ll.state + r.state_off;
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, W, L.in.data, W, ll.big, U, T, U, W, nullptr, nullptr, 0, 1.f, st));
    float * cs = sbase, * ss = sbase + (int64_t) (p.conv - 1) * mamba2_conv_channels(p);
    CAT(CAT_CONV);
    CK(launch_mamba2_conv(ll.big, b, p, L.conv_w.data, L.conv_b.data, cs, ll.slot_floats, ll.xbc, st));
    CAT(CAT_SCAN);
    CK(launch_mamba2_scan(ll.big, ll.xbc, b, p, L.dt_bias.data, L.A_log.data, L.D.data, ss, ll.slot_floats, ll.yssm, st));
    CAT(CAT_NORM);
    CK(launch_mamba2_gate_norm(ll.yssm, ll.big, p, L.gnorm.data, ll.eps, ll.act, ct, T, st));
    CAT(CAT_DENSE);
    return launch_dense(ct, ll.act, inner, L.out.data, inner, out, W, T, W, inner, nullptr, resid, W, 1.f, st);
}
static int mix_decay(pb200_model * m, const BatchView & b, const LRun & r, LLayer & L, const float * resid, float * out) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    const DecayAttnParams & d = L.dec;
    const int QD = d.heads * d.dim, VD = d.heads * d.vdim, C = 2 * QD + 2 * VD;
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, W, L.qkvg.data, W, ll.big, C, T, C, W, nullptr, nullptr, 0, 1.f, st));
    CAT(CAT_SCAN);
    CK(launch_decay_attn(ll.big, C, 0, QD, 2 * QD, b, d, L.decay.data, ll.state + r.state_off, ll.slot_floats, ll.yssm, st));
    CAT(CAT_NORM);
    CK(launch_norm_gate(ll.yssm, ll.big + 2 * QD + VD, C, L.dec_norm_groups, L.dec_norm_weight ? L.onorm.data : nullptr, L.dec_gate_act, ll.eps, ll.act, ct, T, VD, st));
    CAT(CAT_DENSE);
    return launch_dense(ct, ll.act, VD, L.out.data, VD, out, W, T, W, VD, nullptr, resid, W, 1.f, st);
}
static int mix_latent(pb200_model * m, const BatchView & b, bool prefill, const LRun & r, LLayer & L, const float * resid, float * out) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    const LatentParams & a = L.lat;
    const int H = a.heads, C = latent_proj_cols(a), DQ = a.dim + a.rot_dim, VD = H * a.vdim, R = a.kv_rank, RW = latent_row(a);
    float * cache = ll.state + r.state_off;       // this layer's rows, or those of the layer it reads
    const float * gate = ll.big + a.q_rank;
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, W, L.lproj.data, W, ll.big, C, T, C, W, nullptr, nullptr, 0, 1.f, st));
    CAT(CAT_LATENT);
    CK(launch_latent_prep(ll.big, b, a, L.dq_norm.data, L.dkv_norm.data, L.rot_freq.data, ll.eps, ll.act2, ct, cache, ll.slot_floats, st));
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act2, a.q_rank, L.uq.data, a.q_rank, ll.big2, (int64_t) H * DQ, T, H * DQ, a.q_rank, nullptr, nullptr, 0, 1.f, st));
    AttnParams ap;
    ap.heads = H; ap.scale = a.scale;
    AttnIO io;
    CAT(CAT_LATENT);
    if (prefill) {   // keys and values of the batch, expanded from the cached latents
        CK(launch_latent_rope_q(ll.big2, b, a, L.rot_freq.data, st));
        CK(launch_latent_gather(cache, ll.slot_floats, b, a, ll.act2, ct, ll.krb, st));
        CAT(CAT_DENSE);
        if (a.dim > 0) CK(launch_dense(ct, ll.act2, R, L.uk.data, R, ll.big3, (int64_t) H * a.dim, T, H * a.dim, R, nullptr, nullptr, 0, 1.f, st));
        CK(launch_dense(ct, ll.act2, R, L.uv.data, R, ll.big4, VD, T, VD, R, nullptr, nullptr, 0, 1.f, st));
        CAT(CAT_ATTN);
        ap.kv_heads = H; ap.dim = DQ; ap.vdim = a.vdim; ap.shared_dim = a.rot_dim;
        io.q = ll.big2; io.ldq = (int64_t) H * DQ;
        io.k = ll.big3; io.ldk = (int64_t) H * a.dim;
        io.ks = ll.krb; io.ldks = a.rot_dim;
        io.v = ll.big4; io.ldv = VD;
        io.gate = gate; io.ldg = C; io.gate_mode = 2;
        CK(launch_attn_prefill_io(io, b, ap, ll.act, ct, st));
    } else if (T == b.n_entries && R <= 512) {   // one token per entry: the key up-projection folded into the query, rows split over CTAs
        CK(launch_latent_absorb_q(ll.big2, b, L.uk.data, ct, a, L.rot_freq.data, ll.big3, st));
        CAT(CAT_ATTN);
        CK(launch_latent_decode(ll.big3, b, a, cache, ll.slot_floats, latent_decode_splits(a.cache_rows), ll.lat_part, L.uv.data, ct, gate, C, ll.act, ct, st));
    } else {         // the same through the shared decode kernel: one key / value head, the key is the whole row, the value its latent part
        CK(launch_latent_absorb_q(ll.big2, b, L.uk.data, ct, a, L.rot_freq.data, ll.big3, st));
        CAT(CAT_ATTN);
        ap.kv_heads = 1; ap.dim = RW; ap.vdim = R; ap.cache_rows = a.cache_rows;
        io.q = ll.big3; io.ldq = (int64_t) H * RW;
        io.k_row = io.v_row = RW;
        CK(launch_attn_decode_io(io, b, ap, cache, cache, ll.slot_floats, ll.big4, T_F32, st));
        CAT(CAT_LATENT);
        CK(launch_latent_up_v(ll.big4, L.uv.data, ct, a, gate, C, ll.act, ct, T, st));
    }
    CAT(CAT_DENSE);
    return launch_dense(ct, ll.act, VD, L.out.data, VD, out, W, T, W, VD, nullptr, resid, W, 1.f, st);
}

// ---- dual mixer over ll.act: x[t] += mult * join(attention branch, recurrent branch).  JOIN_SCALED_SUM: both branch results, scaled, lie
// side by side in ll.act and ONE output product adds them onto the stream.  JOIN_NORMED_MEAN: each branch has its own output product; the
// two results are normed, averaged and added by one kernel that also leaves rmsnorm(x) * next_norm in ll.act when next_norm is given. ----
static int mix_dual(pb200_model * m, const BatchView & b, bool prefill, const LRun & r, LLayer & L, float * x, float mult, const float * next_norm) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    const AttnParams & a = L.att;
    const DualMix & d = L.dual;
    const GatedLinParams & rp = d.rp;
    const int C = d.cols, OD = a.heads * a.vdim, RV = rp.heads * rp.vdim;
    // the slot's arena for this run: K rows | V rows | convolution inputs | recurrent state
    float * kc = ll.state + r.state_off, * vc = kc + (int64_t) a.cache_rows * a.kv_heads * a.dim;
    int64_t o = (int64_t) a.cache_rows * a.kv_heads * (a.dim + a.vdim);
    o = (o + 3) / 4 * 4;
    float * conv_state = ll.state + r.state_off + o;
    o += (int64_t) std::max(d.taps - 1, 0) * d.conv_ch;
    o = (o + 3) / 4 * 4;
    float * rec_state = ll.state + r.state_off + o;
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, W, L.qkvg.data, W, ll.big, C, T, C, W, nullptr, nullptr, 0, 1.f, st));
    float * src = ll.big;       // where q, k, v of both branches are read from: the projection, or the convolution's output
    int64_t ld = C;
    if (d.taps > 0) {
        CAT(CAT_CONV);
        CK(launch_causal_conv(ll.big, C, b, d.conv_ch, d.taps, L.dconv_w.data, d.conv_l, conv_state, ll.slot_floats, ll.xbc, d.conv_ch, st));
        src = ll.xbc;
        ld = d.conv_ch;
    }
    // ---- attention branch ----
    CAT(CAT_ATTN);
    AttnPrep pr;
    pr.norm = d.qk_norm; pr.wq = L.q_norm.data; pr.wk = L.k_norm.data; pr.eps = ll.eps;
    pr.rot_dims = d.rot_dims; pr.rot_layout = d.rot_layout; pr.rot_freq = L.rot_freq.data;
    pr.v_rot = d.v_rot; pr.v_layout = d.rot_layout; pr.v_freq = d.v_rot ? L.vrot_freq.data : nullptr;
    // one launch prepares both branches: the recurrence's inputs (unit vectors, gates, decays), then the attention inputs and the cache store
    // (PB200_DUAL_UNFUSED: the same steps as the single ops the layers were brought up on, one launch each; for A/B runs and tests)
    static const bool unfused = getenv("PB200_DUAL_UNFUSED") != nullptr;
    if (unfused) {
        if (d.rec == REC_DELTA)
            CK(launch_delta_prep(src + d.c_rq, ld, src + d.c_rk, ld, ll.big + d.c_rb, C, ll.big + d.c_ra, C, L.A_log.data, L.dt_bias.data, rp.qk_heads, rp.heads, rp.dim, T, st));
        else CK(launch_hgrn2_prep(src + d.c_rq, ld, src + d.c_rk, ld, L.f_bias.data, L.f_lower.data, rp.qk_heads * rp.dim, T, st));
        CK(launch_attn_prep_store(src + d.c_q, ld, src + d.c_k, ld, src + d.c_v, ld, b, a, pr, kc, vc, ll.slot_floats, st));
    } else if (d.rec == REC_DELTA)
        CK(launch_dual_prep_store(0, src + d.c_rq, ld, src + d.c_rk, ld, ll.big + d.c_rb, C, ll.big + d.c_ra, C, L.A_log.data, L.dt_bias.data, rp.qk_heads, rp.heads,
                                  rp.dim, src + d.c_q, ld, src + d.c_k, ld, src + d.c_v, ld, b, a, pr, kc, vc, ll.slot_floats, st));
    else
        CK(launch_dual_prep_store(1, src + d.c_rq, ld, src + d.c_rk, ld, nullptr, 0, nullptr, 0, L.f_bias.data, L.f_lower.data, rp.qk_heads, rp.heads, rp.dim,
                                  src + d.c_q, ld, src + d.c_k, ld, src + d.c_v, ld, b, a, pr, kc, vc, ll.slot_floats, st));
    const bool sum = d.join == JOIN_SCALED_SUM;
    // ---- recurrent branch: on the second stream beside the attention branch, unless every launch is being timed ----
    static const bool one_stream = getenv("PB200_ONE_STREAM") != nullptr;   // A/B: both branches in a row on one stream
    const bool forked = !ll.prof_on && !one_stream;
    cudaStream_t rst = st;
    if (forked) {
        if (!ll.side) {
            CK(cudaStreamCreateWithFlags(&ll.side, cudaStreamNonBlocking));
            CK(cudaEventCreateWithFlags(&ll.ev_fork, cudaEventDisableTiming));
            CK(cudaEventCreateWithFlags(&ll.ev_join, cudaEventDisableTiming));
        }
        rst = ll.side;
        CK(cudaEventRecord(ll.ev_fork, st));
        CK(cudaStreamWaitEvent(rst, ll.ev_fork, 0));
    }
    CAT(CAT_SCAN);
    GatedLinIO gi;
    gi.q = src + d.c_rq; gi.ldq = ld;
    gi.v = src + d.c_rv; gi.ldv = ld;
    if (d.rec == REC_DELTA) {
        gi.k = src + d.c_rk; gi.ldk = ld;
        gi.decay = ll.big + d.c_ra; gi.ldd = C;
        gi.beta = ll.big + d.c_rb; gi.ldb = C;
    } else {
        gi.decay = src + d.c_rk; gi.ldd = ld;
    }
    CK(launch_gated_linattn(gi, b, rp, rec_state, ll.slot_floats, ll.yssm, rst));
    if (!sum) {   // every head by its own root mean square with the weight all heads share -> operand of the branch's own output product
        CAT(CAT_NORM);
        CK(launch_norm_gate(ll.yssm, d.rec == REC_DELTA ? ll.big + d.c_rg : nullptr, C, rp.heads, L.onorm.data, d.rec == REC_DELTA ? 1 : -1, ll.eps, ll.act2, ct, T, RV,
                            rst, RV, 1.f));
    }
    if (forked) CK(cudaEventRecord(ll.ev_join, rst));
    // ---- attention branch ----
    CAT(CAT_ATTN);
    AttnIO io;
    io.q = src + d.c_q; io.ldq = ld;
    io.k = src + d.c_k; io.ldk = ld;
    io.v = src + d.c_v; io.ldv = ld;
    io.k_row = (int64_t) a.kv_heads * a.dim; io.v_row = (int64_t) a.kv_heads * a.vdim;
    const bool post = d.v_rot || sum;   // the head results are turned back, gated and scaled into their place by a kernel of their own
    if (!post) { io.gate = ll.big + d.c_g; io.ldg = C; io.gate_mode = d.gate_mode; }
    void * att_out = post ? (void *) ll.big2 : ll.act;
    const int att_type = post ? T_F32 : ct;
    if (prefill) CK(launch_attn_prefill_io(io, b, a, att_out, att_type, st));
    else CK(launch_attn_decode_io(io, b, a, kc, vc, ll.slot_floats, att_out, att_type, st, ll.lat_part));
    const int64_t ldo = sum ? OD + RV : OD;
    if (post && !sum)
        CK(launch_attn_unrotate_gate(ll.big2, b, a.heads, a.vdim, d.rot_layout, d.v_rot ? L.vrot_freq.data : nullptr, ll.big + d.c_g, C, d.gate_mode, 1.f, ll.act,
                                     ldo, ct, st));
    // ---- the branches meet ----
    if (forked) CK(cudaStreamWaitEvent(st, ll.ev_join, 0));
    CAT(CAT_NORM);
    if (sum && unfused) {
        CK(launch_attn_unrotate_gate(ll.big2, b, a.heads, a.vdim, d.rot_layout, d.v_rot ? L.vrot_freq.data : nullptr, ll.big + d.c_g, C, d.gate_mode, d.left_scale,
                                     ll.act, ldo, ct, st));
        CK(launch_norm_gate(ll.yssm, d.rec == REC_DELTA ? ll.big + d.c_rg : nullptr, C, rp.heads, L.onorm.data, d.rec == REC_DELTA ? 1 : -1, ll.eps,
                            (uint8_t *) ll.act + (size_t) OD * esize(ct), ct, T, RV, st, ldo, d.right_scale));
        CAT(CAT_DENSE);
        return launch_dense(ct, ll.act, ldo, L.out.data, ldo, x, W, T, W, (int) ldo, nullptr, x, W, mult, st);
    }
    if (sum) {
        // attention heads turned back and gated; recurrence heads by their own root mean square, the weight all heads share, the SiLU gate; both
        // with their branch's factor, side by side as the operand of the one output product
        CK(launch_dual_post(ll.big2, b, a.heads, a.vdim, d.rot_layout, d.v_rot ? L.vrot_freq.data : nullptr, ll.big + d.c_g, C, d.gate_mode, d.left_scale, ll.yssm,
                            rp.heads, rp.vdim, d.rec == REC_DELTA ? ll.big + d.c_rg : nullptr, C, L.onorm.data, d.rec == REC_DELTA ? 1 : -1, ll.eps, d.right_scale,
                            ll.act, ldo, ct, st));
        CAT(CAT_DENSE);
        return launch_dense(ct, ll.act, ldo, L.out.data, ldo, x, W, T, W, (int) ldo, nullptr, x, W, mult, st);
    }
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, OD, L.out.data, OD, ll.big4, 2 * W, T, W, OD, nullptr, nullptr, 0, 1.f, st));
    CK(launch_dense(ct, ll.act2, RV, L.out_r.data, RV, ll.big4 + W, 2 * W, T, W, RV, nullptr, nullptr, 0, 1.f, st));
    CAT(CAT_NORM);
    return launch_rmsnorm_pair_residual(ll.big4, 2 * W, ll.big4 + W, 2 * W, L.join_wl.data, L.join_wr.data, mult * d.left_scale, ll.eps, x, next_norm,
                                        next_norm ? ll.act : nullptr, ct, T, W, st);
}

// ---- clamped gated feed-forward: x[t] += down(glu(gateup(ll.act[t]))); ll.act stays as it is ----
static int ff_clamped(pb200_model * m, int T, const DenseW & gateup, const DenseW & down, int ff, float limit, float * x) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int W = ll.width, ct = ll.ctype;
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, W, gateup.data, W, ll.big, 2 * ff, T, 2 * ff, W, nullptr, nullptr, 0, 1.f, st));
    CAT(CAT_ELEM);
    CK(launch_clamped_glu(ll.big, ll.act2, ct, T, ff, limit, st));
    CAT(CAT_DENSE);
    return launch_dense(ct, ll.act2, ff, down.data, ff, x, W, T, W, ff, nullptr, x, W, 1.f, st);
}
// ---- squared-ReLU feed-forward: out[t] = down(max(up(ll.act[t]), 0)^2); ll.act stays as it is ----
static int ff_relu2(pb200_model * m, int T, const DenseW & up, const DenseW & down, int ff, float * out) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int W = ll.width, ct = ll.ctype;
    CAT(CAT_DENSE);
    CK(launch_dense(ct, ll.act, W, up.data, W, ll.big, ff, T, ff, W, nullptr, nullptr, 0, 1.f, st));
    CAT(CAT_ELEM);
    CK(launch_relu2(ll.big, ll.act2, ct, (int64_t) T * ff, st));
    CAT(CAT_DENSE);
    return launch_dense(ct, ll.act2, ff, down.data, ff, out, W, T, W, ff, nullptr, nullptr, 0, 1.f, st);
}
// ---- mixture of experts over ll.act.  accumulate: x[t] += shared(h) + sum_k w_k expert_k(h) (the stream itself); otherwise x receives the
// sublayer's result alone.  The router form and the expert form come from the layer (LLayer::route, MoeParams::act). ----
static int ff_moe(pb200_model * m, int T, bool prefill, LLayer & L, float * x, bool accumulate, float out_scale = 1.f) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int W = ll.width, ct = ll.ctype;
    const MoeParams & p = L.moe;
    const size_t es = esize(ct);
    const int UR = moe_up_rows(p);
    int base = MOE_ADD;
    const float * xscale = nullptr;
    CAT(CAT_MOE);
    if (L.route == ROUTE_SIGMOID_GROUPS) {
        CK(launch_moe_route_sigmoid(ll.act, ct, L.router.data, L.router_b.data, p, W, L.shared_ff > 0 ? L.shared_gate.data : nullptr, ll.moe_idx, ll.moe_wt, ll.moe_sg, T, st));
        if (accumulate) return PB200_ENOTSUP;
        if (L.shared_ff > 0) {   // the shared expert's result waits in x; the kernel that sums the experts multiplies it by the token's gate
            if (p.act == 1) CK(ff_relu2(m, T, L.s_gateup, L.s_down, L.shared_ff, x));
            else return PB200_ENOTSUP;
            base = MOE_SCALE;
            xscale = ll.moe_sg;
        } else {
            base = MOE_SET;
        }
    } else if (L.route == ROUTE_SIGMOID_PLAIN) {   // plain sigmoid scores: no correction, no groups, the chosen scores are the weights
        CK(launch_moe_route_sigmoid(ll.act, ct, L.router.data, nullptr, p, W, nullptr, ll.moe_idx, ll.moe_wt, nullptr, T, st));
        if (L.shared_ff > 0 || p.act != 2) return PB200_ENOTSUP;
        if (!accumulate) base = MOE_SET;
    } else {
        CK(launch_moe_route(ll.act, ct, L.router.data, L.router_b.data, p, W, ll.moe_idx, ll.moe_wt, T, st));
        if (!accumulate || p.act != 0) return PB200_ENOTSUP;
        if (L.shared_ff > 0) CK(ff_clamped(m, T, L.s_gateup, L.s_down, L.shared_ff, L.shared_limit, x));
    }
    // a weight on the expert's input rides on the gate / up products; the sum over the experts then takes none
    const float * in_wt = p.weight_on_input ? ll.moe_wt : nullptr, * sum_wt = p.weight_on_input ? nullptr : ll.moe_wt;
    auto activate = [&](int rows) -> int {
        if (p.act == 1) return launch_relu2(ll.moe_gu, ll.moe_y, ct, (int64_t) rows * p.ff, st);
        if (p.act == 2) return launch_silu_mul(ll.moe_gu, ll.moe_y, ct, rows, p.ff, in_wt, ll.moe_perm, st);
        return launch_clamped_glu(ll.moe_gu, ll.moe_y, ct, rows, p.ff, p.limit, st);
    };
    CAT(CAT_MOE);
    if (!prefill || (int64_t) T * p.top <= 64) {
        CK(launch_moe_gateup_rows(ll.act, ct, L.e_gateup.data, ll.moe_idx, p, W, ll.moe_y, T, st, in_wt));
        return launch_moe_down_rows(ll.moe_y, ct, L.e_down.data, ll.moe_idx, sum_wt, p, W, x, T, st, base, xscale, out_scale);
    }
    const int P = T * p.top, E = p.experts;
    CK(launch_moe_sort(ll.moe_idx, p, T, ll.moe_count, ll.moe_start, ll.moe_perm, st));
    CK(launch_moe_gather(ll.act, ct, ll.moe_perm, p.top, W, ll.moe_hs, P, st));
    if (dense_grouped_ok(ct, UR, W, W, W, (int64_t) UR * W, ll.moe_hs, L.e_gateup.data) &&
        dense_grouped_ok(ct, W, p.ff, p.ff, p.ff, (int64_t) W * p.ff, ll.moe_y, L.e_down.data)) {
        // all experts in one launch each way; the row counts never leave the device
        CK(launch_dense_grouped(ct, ll.moe_hs, W, L.e_gateup.data, W, (int64_t) UR * W, ll.moe_gu, UR, ll.moe_start, ll.moe_count, E, P, UR, W, st));
        CK(activate(P));
        CK(launch_dense_grouped(ct, ll.moe_y, p.ff, L.e_down.data, p.ff, (int64_t) W * p.ff, ll.moe_ds, W, ll.moe_start, ll.moe_count, E, P, W, p.ff, st));
        return launch_moe_combine(ll.moe_ds, ll.moe_perm, ll.moe_row_of, sum_wt, p.top, W, x, T, st, base, xscale, out_scale);
    }
    CK(cudaMemcpyAsync(ll.moe_count_host, ll.moe_count, (size_t) E * 4, cudaMemcpyDeviceToHost, st));
    CK(cudaMemcpyAsync(ll.moe_count_host + 4096, ll.moe_start, (size_t) E * 4, cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));   // the per-expert row counts size the products below
    const int32_t * cnt = ll.moe_count_host, * start = ll.moe_count_host + 4096;
    for (int e = 0; e < E; e++)
        if (cnt[e] > 0)
            CK(launch_dense(ct, (const uint8_t *) ll.moe_hs + (size_t) start[e] * W * es, W, (const uint8_t *) L.e_gateup.data + (size_t) e * UR * W * es, W,
                            ll.moe_gu + (int64_t) start[e] * UR, UR, cnt[e], UR, W, nullptr, nullptr, 0, 1.f, st));
    CK(activate(P));
    for (int e = 0; e < E; e++)
        if (cnt[e] > 0)
            CK(launch_dense(ct, (const uint8_t *) ll.moe_y + (size_t) start[e] * p.ff * es, p.ff, (const uint8_t *) L.e_down.data + (size_t) e * W * p.ff * es, p.ff,
                            ll.moe_ds + (int64_t) start[e] * W, W, cnt[e], W, p.ff, nullptr, nullptr, 0, 1.f, st));
    return launch_moe_combine(ll.moe_ds, ll.moe_perm, ll.moe_row_of, sum_wt, p.top, W, x, T, st, base, xscale, out_scale);
}

// FRAME_POSTNORM: the stream starts as embedding + position vector; x <- x + mult * LN(mixer(x)), x <- x + mult * LN(ff(x)) with weight
// and bias in LN; the sublayers read x itself (ll.act holds it in the operand type, written by the kernel that updated x).
static int ll_forward_postnorm(pb200_model * m, const BatchView & b, bool prefill, const int32_t * tokens_dev, const int32_t * want_dev, int nW, int lrow0) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    CAT(CAT_ELEM);
    CK(launch_embed_pos(ll.embed.data, ll.pos_table.data, ct, W, tokens_dev, b, ll.x, ll.act, ct, st));
    for (size_t ir = 0; ir < ll.runs.size(); ir++) {
        const LRun & r = ll.runs[ir];
        LLayer & L = ll.layers[(size_t) r.layer];
        const bool last = ir + 1 == ll.runs.size();
        if (L.kind != MIX_ATTENTION) return PB200_ENOTSUP;
        CK(mix_attention(m, b, prefill, r, L, nullptr, ll.msub));
        CAT(CAT_NORM);
        CK(launch_layernorm_affine_residual(ll.msub, L.norm1.data, L.norm1_bias.data, ll.resid_mult, ll.eps, ll.x, (last && L.ff <= 0) ? nullptr : ll.act, ct, T, W, st));
        if (L.ff > 0) {
            if (L.ff_kind == FF_MOE) CK(ff_moe(m, T, prefill, L, ll.msub, false));
            else if (L.ff_kind == FF_RELU2) CK(ff_relu2(m, T, L.gateup, L.down, L.ff, ll.msub));
            else return PB200_ENOTSUP;
            CAT(CAT_NORM);
            CK(launch_layernorm_affine_residual(ll.msub, L.norm2.data, L.norm2_bias.data, ll.resid_mult, ll.eps, ll.x, last ? nullptr : ll.act, ct, T, W, st));
        }
        if (ll.tap_on) CK(cudaMemcpyAsync(ll.tap + (int64_t) ir * T * W, ll.x, (size_t) T * W * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (nW > 0) {
        CAT(CAT_HEAD);
        CK(launch_layernorm_affine(ll.x, want_dev, ll.final_norm.data, ll.final_norm_bias.data, ll.eps, ll.actw, ct, nW, W, st));
        float * lg = ll.logits + (int64_t) lrow0 * ll.vocab;
        CK(launch_dense(ct, ll.actw, W, ll.head.data, W, lg, ll.vocab, nW, ll.vocab, W, nullptr, nullptr, 0, ll.logit_scale, st));
        CK(launch_softcap(lg, (int64_t) nW * ll.vocab, ll.logit_softcap, st));
    }
    CAT(-1);
    return 0;
}

// FRAME_PRERMS: the stream starts as embed * scale + bigram row; x <- x + mult * mixer(norm1 x), x <- x + mult * ff(norm2 x) with RMS norms of
// one learned number (kept as a constant vector); every pass of the repeated block first adds the embedding output (not the first pass) and
// its step vector.  ll.act holds the next sublayer's normed input in the operand type.
static int ll_forward_prerms(pb200_model * m, const BatchView & b, bool prefill, const int32_t * tokens_dev, const int32_t * want_dev, int nW, int lrow0) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    CAT(CAT_ELEM);
    CK(launch_embed_bigram(ll.embed.data, ll.bigram.buckets > 0 ? ll.bigram_table.data : nullptr, ct, W, ll.embed_scale, ll.bigram, tokens_dev, b, ll.x,
                           ll.loop_times > 1 ? ll.x0 : nullptr, st));
    bool act_ready = false;   // the kernel that closed the previous sublayer has left this one's normed input in ll.act
    for (size_t ir = 0; ir < ll.runs.size(); ir++) {
        const LRun & r = ll.runs[ir];
        LLayer & L = ll.layers[(size_t) r.layer];
        if (L.kind != MIX_DUAL) return PB200_ENOTSUP;
        if (r.pass >= 0) {
            CAT(CAT_NORM);
            CK(launch_stream_add_rmsnorm(ll.x, r.pass > 0 ? ll.x0 : nullptr, ll.loop_step.data + (int64_t) r.pass * W, L.norm1.data, ll.eps, ll.act, ct, T, W, st));
        } else if (!act_ready) {
            CAT(CAT_NORM);
            CK(launch_group_rmsnorm(ll.x, nullptr, L.norm1.data, 1, ll.eps, ll.act, ct, T, W, st));
        }
        act_ready = false;
        // the norm that follows the mixer: this layer's second one, or the next run's first one unless that run opens a pass
        const float * next_norm = nullptr;
        if (L.ff > 0) next_norm = L.norm2.data;
        else if (ir + 1 < ll.runs.size() && ll.runs[ir + 1].pass < 0) next_norm = ll.layers[(size_t) ll.runs[ir + 1].layer].norm1.data;
        CK(mix_dual(m, b, prefill, r, L, ll.x, ll.resid_mult, next_norm));
        const bool fused = L.dual.join == JOIN_NORMED_MEAN && next_norm;
        if (L.ff > 0) {
            if (!fused) {
                CAT(CAT_NORM);
                CK(launch_group_rmsnorm(ll.x, nullptr, L.norm2.data, 1, ll.eps, ll.act, ct, T, W, st));
            }
            if (L.ff_kind != FF_MOE) return PB200_ENOTSUP;
            CK(ff_moe(m, T, prefill, L, ll.x, true, ll.resid_mult));
        } else {
            act_ready = fused;
        }
        if (ll.tap_on) CK(cudaMemcpyAsync(ll.tap + (int64_t) ir * T * W, ll.x, (size_t) T * W * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (nW > 0) {
        CAT(CAT_HEAD);
        CK(launch_group_rmsnorm(ll.x, want_dev, ll.final_norm.data, 1, ll.eps, ll.actw, ct, nW, W, st));
        CK(launch_dense(ct, ll.actw, W, ll.head.data, W, ll.logits + (int64_t) lrow0 * ll.vocab, ll.vocab, nW, ll.vocab, W, nullptr, nullptr, 0, ll.logit_scale, st));
    }
    CAT(-1);
    return 0;
}

// FRAME_PRENORM: x <- x + mixer(shift(norm1 x)), x <- x + ff(norm2 x), then the weighted sum over the embedding output and the results
// of all layers so far goes on.  ll.hist plane j holds X_j; ll.x the stream that enters the next layer.
static int ll_forward_prenorm(pb200_model * m, const BatchView & b, bool prefill, const int32_t * tokens_dev, const int32_t * want_dev, int nW, int lrow0) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype, G = ll.norm_groups;
    const int64_t plane = (int64_t) ll.capT * W;
    CAT(CAT_ELEM);
    CK(launch_embed(ll.embed.data, ct, W, tokens_dev, T, ll.x, ll.hist, st));
    bool act_ready = false;   // the kernel that closed the previous layer has left this layer's mixer input in ll.act
    for (size_t ir = 0; ir < ll.runs.size(); ir++) {
        const LRun & r = ll.runs[ir];
        LLayer & L = ll.layers[(size_t) r.layer];
        float * xn = ll.hist + (int64_t) (ir + 1) * plane;
        if (!act_ready) {
            CAT(CAT_NORM);
            CK(launch_group_rmsnorm_shift(ll.x, b, L.norm1.data, G, ll.eps, L.shift.data, ll.state + r.shift_off, ll.slot_floats, ll.act, ct, W, st));
        }
        act_ready = false;
        if (L.kind == MIX_DECAY) CK(mix_decay(m, b, r, L, ll.x, xn));
        else if (L.kind == MIX_LATENT) CK(mix_latent(m, b, prefill, r, L, ll.x, xn));
        else if (L.kind == MIX_ATTENTION) CK(mix_attention(m, b, prefill, r, L, ll.x, xn));
        else CK(mix_mamba2(m, b, r, L, ll.x, xn));
        if (L.ff > 0) {
            CAT(CAT_NORM);
            CK(launch_group_rmsnorm(xn, nullptr, L.norm2.data, G, ll.eps, ll.act, ct, T, W, st));
            if (L.ff_kind == FF_MOE) CK(ff_moe(m, T, prefill, L, xn, true));
            else CK(ff_clamped(m, T, L.gateup, L.down, L.ff, L.ff_limit, xn));
        }
        if (b.max_n == 1 && ir + 1 < ll.runs.size()) {   // one-token entries: the depth average and the next layer's norm + shift in one kernel
            const LRun & rn = ll.runs[ir + 1];
            const LLayer & Ln = ll.layers[(size_t) rn.layer];
            CAT(CAT_NORM);
            CK(launch_depth_average_norm_shift(ll.hist, plane, L.dwa.data, (int) ir + 2, ll.x, b, Ln.norm1.data, G, ll.eps, Ln.shift.data, ll.state + rn.shift_off,
                                               ll.slot_floats, ll.act, ct, W, st));
            act_ready = true;
        } else {
            CAT(CAT_ELEM);
            CK(launch_depth_average(ll.hist, plane, L.dwa.data, (int) ir + 2, ll.x, (int64_t) T * W, st));
        }
        if (ll.tap_on) CK(cudaMemcpyAsync(ll.tap + (int64_t) ir * T * W, ll.x, (size_t) T * W * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (nW > 0) {
        CAT(CAT_HEAD);
        CK(launch_group_rmsnorm(ll.x, want_dev, ll.final_norm.data, G, ll.eps, ll.actw, ct, nW, W, st));
        CK(launch_dense(ct, ll.actw, W, ll.head.data, W, ll.logits + (int64_t) lrow0 * ll.vocab, ll.vocab, nW, ll.vocab, W, nullptr, nullptr, 0, ll.logit_scale, st));
    }
    CAT(-1);
    return 0;
}

static int ll_forward(pb200_model * m, const BatchView & b, bool prefill, const int32_t * tokens_dev, const int32_t * want_dev, int nW, int lrow0) {
    LayerList & ll = *m->ll;
    cudaStream_t st = m->stream;
    ll.prof_cat.clear();
    CK(tap_prepare(m, b.n_tokens));
    if (ll.frame == FRAME_PRENORM) return ll_forward_prenorm(m, b, prefill, tokens_dev, want_dev, nW, lrow0);
    if (ll.frame == FRAME_POSTNORM) return ll_forward_postnorm(m, b, prefill, tokens_dev, want_dev, nW, lrow0);
    if (ll.frame == FRAME_PRERMS) return ll_forward_prerms(m, b, prefill, tokens_dev, want_dev, nW, lrow0);
    CAT(CAT_ELEM);
    const int T = b.n_tokens, W = ll.width, ct = ll.ctype;
    CK(launch_embed(ll.embed.data, ct, W, tokens_dev, T, ll.x, ll.x0, st));
    float * x = ll.x, * xalt = ll.xalt;
    bool act_ready = false;
    for (size_t ir = 0; ir < ll.runs.size(); ir++) {
        const LRun & r = ll.runs[ir];
        LLayer & L = ll.layers[(size_t) r.layer];
        if (r.pass >= 0) {
            // x <- W_in [x ; x0] + step[pass]: two products over the halves of W_in, the second accumulating onto the first
            CAT(CAT_ELEM);
            CK(launch_cast(x, ll.act, ct, (int64_t) T * W, st));
            CK(launch_cast(ll.x0, ll.act2, ct, (int64_t) T * W, st));
            CAT(CAT_DENSE);
            CK(launch_dense(ct, ll.act, W, ll.loop_in.data, 2 * W, xalt, W, T, W, W, ll.loop_step.data + (int64_t) r.pass * W, nullptr, 0, 1.f, st));
            CK(launch_dense(ct, ll.act2, W, (const uint8_t *) ll.loop_in.data + (size_t) W * esize(ct), 2 * W, xalt, W, T, W, W, nullptr, xalt, W, 1.f, st));
            std::swap(x, xalt);
        }
        if (!act_ready) {   // otherwise the previous run's closing norm has already left layernorm(x) * norm1 in ll.act
            CAT(CAT_NORM);
            CK(launch_layernorm(x, nullptr, L.norm1.data, ll.eps, ll.act, ct, T, W, st));
        }
        act_ready = false;
        // the norm that closes this run also opens the next one, unless a pass of the repeated block (its input mix) or the end comes first
        const LLayer * nextL = (ir + 1 < ll.runs.size() && ll.runs[ir + 1].pass < 0) ? &ll.layers[(size_t) ll.runs[ir + 1].layer] : nullptr;
        if (L.kind == MIX_ATTENTION) CK(mix_attention(m, b, prefill, r, L, nullptr, ll.msub));
        else if (L.kind == MIX_MAMBA2) CK(mix_mamba2(m, b, r, L, nullptr, ll.msub));
        else if (L.kind == MIX_DECAY) CK(mix_decay(m, b, r, L, nullptr, ll.msub));
        else CK(mix_latent(m, b, prefill, r, L, nullptr, ll.msub));
        CAT(CAT_NORM);
        if (L.ff > 0) CK(launch_layernorm_residual_next(ll.msub, L.norm1b.data, L.norm2.data, ll.eps, x, ll.act, ct, T, W, st));
        else if (nextL) { CK(launch_layernorm_residual_next(ll.msub, L.norm1b.data, nextL->norm1.data, ll.eps, x, ll.act, ct, T, W, st)); act_ready = true; }
        else CK(launch_layernorm_residual(ll.msub, L.norm1b.data, ll.eps, x, T, W, st));
        if (L.ff > 0) {
            CAT(CAT_DENSE);
            CK(launch_dense(ct, ll.act, W, L.gateup.data, W, ll.big, 2 * L.ff, T, 2 * L.ff, W, nullptr, nullptr, 0, 1.f, st));
            CAT(CAT_ELEM);
            CK(launch_gelu_mul(ll.big, ll.act, ct, T, L.ff, st));
            CAT(CAT_DENSE);
            CK(launch_dense(ct, ll.act, L.ff, L.down.data, L.ff, ll.msub, W, T, W, L.ff, nullptr, nullptr, 0, 1.f, st));
            CAT(CAT_NORM);
            if (nextL) { CK(launch_layernorm_residual_next(ll.msub, L.norm2b.data, nextL->norm1.data, ll.eps, x, ll.act, ct, T, W, st)); act_ready = true; }
            else CK(launch_layernorm_residual(ll.msub, L.norm2b.data, ll.eps, x, T, W, st));
        }
        if (ll.tap_on) CK(cudaMemcpyAsync(ll.tap + (int64_t) ir * T * W, x, (size_t) T * W * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (nW > 0) {
        CAT(CAT_HEAD);
        CK(launch_layernorm(x, want_dev, ll.final_norm.data, ll.eps, ll.actw, ct, nW, W, st));
        CK(launch_dense(ct, ll.actw, W, ll.head.data, W, ll.logits + (int64_t) lrow0 * ll.vocab, ll.vocab, nW, ll.vocab, W, nullptr, nullptr, 0, ll.logit_scale, st));
    }
    CAT(-1);
    return 0;
}
static int prof_collect(pb200_model * m) {   // after the stream has been synchronised
    LayerList & ll = *m->ll;
    if (!ll.prof_on) return 0;
    for (int c = 0; c < 10; c++) ll.prof_ms[c] = 0.f;
    for (size_t i = 0; i + 1 < ll.prof_cat.size(); i++) {
        float ms = 0.f;
        CK(cudaEventElapsedTime(&ms, ll.prof_ev[i], ll.prof_ev[i + 1]));
        if (ll.prof_cat[i] >= 0) ll.prof_ms[ll.prof_cat[i]] += ms;
        ll.prof_ms[CAT_TOTAL] += ms;
    }
    return 0;
}

// builds the device metadata of one homogeneous batch and runs it
struct SubEntry { int slot, n, pos0; const int32_t * tokens; std::vector<std::pair<int, int>> want; /* (local token index, logits row) */ };

static int ll_run_sub(pb200_model * m, std::vector<SubEntry> & es, bool prefill) {
    LayerList & ll = *m->ll;
    const int nE = (int) es.size();
    if (!nE) return 0;
    int T = 0, nW = 0, max_n = 0;
    for (const SubEntry & e : es) { T += e.n; nW += (int) e.want.size(); max_n = std::max(max_n, e.n); }
    CK(ll_reserve(m, T, nW, nE));
    // meta layout: tokens[T] | entry_of[T] | slot[nE] | off[nE+1] | pos0[nE] | want[nW] | prev[nE]
    int32_t * h = ll.meta_host;
    int32_t *h_tok = h, *h_ent = h + T, *h_slot = h + 2 * T, *h_off = h_slot + nE, *h_pos = h_off + nE + 1, *h_want = h_pos + nE;
    int t = 0;
    std::vector<int> lrows;
    for (int i = 0; i < nE; i++) {
        const SubEntry & e = es[(size_t) i];
        h_slot[i] = e.slot; h_off[i] = t; h_pos[i] = e.pos0;
        for (int k = 0; k < e.n; k++) { h_tok[t + k] = e.tokens[k]; h_ent[t + k] = i; }
        t += e.n;
    }
    h_off[nE] = t;
    // wanted rows: logits rows must be contiguous per call of the head product, so they are computed into a staging order and scattered on the host side
    int w = 0;
    for (int i = 0; i < nE; i++)
        for (const auto & pr : es[(size_t) i].want) { h_want[w++] = h_off[i] + pr.first; lrows.push_back(pr.second); }
    int32_t * h_prev = h_want + nW;   // the token before each entry's first one (-1: none)
    for (int i = 0; i < nE; i++) h_prev[i] = es[(size_t) i].pos0 > 0 ? ll.seq_prev[(size_t) es[(size_t) i].slot] : -1;
    const size_t total = (size_t) (h_prev + nE - h);
    int32_t * d = ll.meta_dev;
    CK(cudaMemcpyAsync(d, h, total * 4, cudaMemcpyHostToDevice, m->stream));
    BatchView b;
    b.n_entries = nE; b.n_tokens = T; b.max_n = max_n;
    b.slot = d + 2 * T; b.off = b.slot + nE; b.pos0 = b.off + nE + 1; b.entry_of = d + T; b.prev = d + (h_prev - h);
    static const bool no_graph = getenv("PB200_NO_STEP_GRAPH") != nullptr;
    bool ran = false;
    if (!prefill && m->use_graph && !no_graph && !ll.tap_on && !ll.prof_on && T == nE) {
        LayerList::StepGraph & g = ll.graphs[((uint64_t) nE << 32) | (uint32_t) nW];
        if (!g.exec && g.seen >= 1 && ll.graphs.size() <= 256) {   // second step of this shape: capture (the first one ran directly and set kernel attributes)
            cudaGraph_t graph = nullptr;
            const uint64_t l0 = g_launches.load();
            if (cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
                const int rc = ll_forward(m, b, false, d, d + (h_want - h), nW, 0);
                const cudaError_t ce = cudaStreamEndCapture(m->stream, &graph);
                if (rc == 0 && ce == cudaSuccess && graph && cudaGraphInstantiate(&g.exec, graph, 0) == cudaSuccess) g.launches = g_launches.load() - l0;
                else g.exec = nullptr;
                if (graph) cudaGraphDestroy(graph);
            }
            cudaGetLastError();   // a failed capture must not poison later calls: direct launches below
            g_launches -= g_launches.load() - l0;
        }
        g.seen++;
        if (g.exec) {
            CK(cudaGraphLaunch(g.exec, m->stream));
            g_launches += g.launches;
            ran = true;
        }
    }
    if (!ran) CK(ll_forward(m, b, prefill, d, d + (h_want - h), nW, 0));
    if (nW > 0) CK(cudaMemcpyAsync(ll.logits_host, ll.logits, (size_t) nW * ll.vocab * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    CK(prof_collect(m));
    // hand the rows to the caller's order
    for (int i = 0; i < nE; i++) {
        const SubEntry & e = es[(size_t) i];
        ll.seq_len[(size_t) e.slot] = e.pos0 + e.n;
        ll.seq_prev[(size_t) e.slot] = e.tokens[e.n - 1];
    }
    ll.rows_tmp.assign(lrows.begin(), lrows.end());
    return 0;
}

int ll_batch_step(pb200_model * m, int n_entries, const pb200_batch_entry * entries, float * logits_out, int32_t * greedy_out) {
    LayerList & ll = *m->ll;
    if (!m->finalized) return PB200_ESTATE;
    if (n_entries <= 0 || !entries) return PB200_EINVAL;
    cudaSetDevice(m->device);
    // validate, assign logits rows in entry order
    std::vector<int> row_base((size_t) n_entries);
    int rows = 0;
    for (int i = 0; i < n_entries; i++) {
        const pb200_batch_entry & e = entries[i];
        if (e.seq < 0 || e.seq >= ll.n_seq || ll.seq_len[(size_t) e.seq] < 0 || e.n_tokens <= 0 || !e.tokens || e.n_want < 0 || (e.n_want > 0 && !e.want)) return PB200_EINVAL;
        for (int j = 0; j < i; j++)
            if (entries[j].seq == e.seq) return PB200_EINVAL;
        for (int k = 0; k < e.n_tokens; k++)
            if (e.tokens[k] < 0 || e.tokens[k] >= ll.vocab) return PB200_EINVAL;
        for (int k = 0; k < e.n_want; k++)
            if (e.want[k] < 0 || e.want[k] >= e.n_tokens) return PB200_EINVAL;
        if (ll.ctx_limited && ll.seq_len[(size_t) e.seq] + e.n_tokens > ll.n_ctx) return PB200_EINVAL;
        if (ll.max_pos > 0 && ll.seq_len[(size_t) e.seq] + e.n_tokens > ll.max_pos) return PB200_EINVAL;   // no position vector beyond the table
        row_base[(size_t) i] = rows;
        rows += e.n_want;
    }
    const bool want_greedy = greedy_out != nullptr;
    const int V = ll.vocab;
    auto deliver = [&](float * dst_rows_base) {
        for (size_t k = 0; k < ll.rows_tmp.size(); k++) {
            const int row = ll.rows_tmp[k];
            if (row >= 0 && dst_rows_base) memcpy(dst_rows_base + (size_t) row * V, ll.logits_host + k * V, (size_t) V * 4);
        }
    };
    // greedy tokens need the logits of every entry's last token; they ride as extra wanted rows (row index < 0 encodes the entry)
    auto take_greedy = [&]() {
        for (size_t k = 0; k < ll.rows_tmp.size(); k++) {
            const int row = ll.rows_tmp[k];
            if (row < 0) greedy_out[-row - 1] = ll.greedy_host[k];
        }
    };
    auto run = [&](std::vector<SubEntry> & sub, bool prefill) -> int {
        if (sub.empty()) return 0;
        CK(ll_run_sub(m, sub, prefill));
        if (want_greedy && !ll.rows_tmp.empty()) {
            const int nW = (int) ll.rows_tmp.size();
            CK(launch_argmax_rows(ll.logits, V, nW, ll.greedy_dev, m->stream));
            CK(cudaMemcpyAsync(ll.greedy_host, ll.greedy_dev, (size_t) nW * 4, cudaMemcpyDeviceToHost, m->stream));
            CK(cudaStreamSynchronize(m->stream));
            take_greedy();
        }
        deliver(logits_out);
        return 0;
    };
    // 1) entries that start a sequence go through together as one prompt batch
    std::vector<SubEntry> sub;
    for (int i = 0; i < n_entries; i++) {
        const pb200_batch_entry & e = entries[i];
        if (ll.seq_len[(size_t) e.seq] != 0) continue;
        SubEntry s{e.seq, e.n_tokens, 0, e.tokens, {}};
        for (int k = 0; k < e.n_want; k++) s.want.emplace_back(e.want[k], row_base[(size_t) i] + k);
        if (want_greedy) s.want.emplace_back(e.n_tokens - 1, -(i + 1));
        sub.push_back(std::move(s));
    }
    std::vector<char> done((size_t) n_entries, 0);
    for (int i = 0; i < n_entries; i++) done[(size_t) i] = ll.seq_len[(size_t) entries[i].seq] == 0;
    CK(run(sub, true));
    // 2) entries that continue a sequence advance one token per pass, all of them in one batch per pass
    int max_n = 0;
    for (int i = 0; i < n_entries; i++)
        if (!done[(size_t) i]) max_n = std::max(max_n, entries[i].n_tokens);
    for (int k = 0; k < max_n; k++) {
        sub.clear();
        for (int i = 0; i < n_entries; i++) {
            const pb200_batch_entry & e = entries[i];
            if (done[(size_t) i] || e.n_tokens <= k) continue;
            SubEntry s{e.seq, 1, ll.seq_len[(size_t) e.seq], e.tokens + k, {}};
            for (int j = 0; j < e.n_want; j++)
                if (e.want[j] == k) s.want.emplace_back(0, row_base[(size_t) i] + j);
            if (want_greedy && k == e.n_tokens - 1) s.want.emplace_back(0, -(i + 1));
            sub.push_back(std::move(s));
        }
        CK(run(sub, false));
    }
    return 0;
}

int ll_debug_read(pb200_model * m, const char * name, float * host, int64_t n) {
    LayerList & ll = *m->ll;
    cudaSetDevice(m->device);
    CK(cudaStreamSynchronize(m->stream));
    if (strcmp(name, "profile") == 0) {   // ms of the last batch: dense, attention, convolution, scan, norms, element-wise, head, [7] = total,
        if (n > 10) return PB200_EINVAL;   // [8] = routed experts, [9] = the small steps around latent attention (norm + rotation, gather, folds)
        memcpy(host, ll.prof_ms, (size_t) n * 4);
        return 0;
    }
    if (strcmp(name, "layers") == 0) {
        if (!ll.tap || n > ll.tap_floats) return PB200_EINVAL;
        return (int) cudaMemcpy(host, ll.tap, (size_t) n * 4, cudaMemcpyDeviceToHost);
    }
    return PB200_EINVAL;
}

// ---------------------------------------------------------------------------------------------------------------
extern "C" {

int pb200_arch_count(void) { return arch_count(); }
const char * pb200_arch_name(int i) { const ArchEntry * a = arch_at(i); return a ? a->name : nullptr; }
int pb200_arch_family(const char * name) { const ArchEntry * a = arch_find(name); return a ? a->family : -1; }

pb200_model * pb200_model_create_from_config(const char * config_json, int compute_type, int device, int n_ctx, int n_seq) {
    if (!config_json || (compute_type != T_F32 && compute_type != T_BF16) || n_ctx <= 0 || n_seq > 4096) return nullptr;
    Json cfg;
    if (!json_parse(config_json, cfg) || cfg.kind != Json::OBJ) return nullptr;
    const ArchEntry * arch = arch_find(cfg.string("architecture").c_str());
    if (!arch || arch->family != ARCH_LAYERS) return nullptr;
    LayerList * ll = new LayerList();
    ll->arch = arch;
    ll->ctype = compute_type;
    ll->n_ctx = n_ctx;
    ll->n_seq = n_seq;
    std::string err;
    if (arch->configure(cfg, *ll, err) != 0) {
        fprintf(stderr, "[pb200] %s configuration: %s\n", arch->name, err.c_str());
        delete ll;
        return nullptr;
    }
    if (cudaSetDevice(device) != cudaSuccess) { delete ll; return nullptr; }
    pb200_model * m = new pb200_model();
    m->ll = ll;
    m->device = device;
    m->with_embd = m->with_head = true;
    m->hp.n_layer = (int32_t) ll->layers.size();
    m->hp.n_embd = ll->width;
    m->hp.n_vocab = ll->vocab;
    m->hp.n_ctx = n_ctx;
    m->l0 = 0;
    m->l1 = m->hp.n_layer;
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) { delete ll; delete m; return nullptr; }
    if (ll_alloc_params(m) != 0) { pb200_model_free(m); return nullptr; }
    return m;
}

// config.json + model.safetensors of a directory -> finalized model.  A safetensors file is an 8-byte little-endian header length, a JSON
// table name -> {dtype, shape, data_offsets}, then the tensor data; the file is mapped and every tensor handed to pb200_model_set_tensor.
int pb200_model_load_dir(const char * dir, int compute_type, int device, int n_ctx, int n_seq, pb200_model ** out) {
    if (!dir || !out) return PB200_EINVAL;
    *out = nullptr;
    const std::string d(dir);
    std::string cfg_text;
    {
        FILE * f = fopen((d + "/config.json").c_str(), "rb");
        if (!f) return PB200_EINVAL;
        char buf[4096];
        size_t n;
        while ((n = fread(buf, 1, sizeof buf, f)) > 0) cfg_text.append(buf, n);
        fclose(f);
    }
    Json cfg;
    if (!json_parse(cfg_text, cfg) || cfg.kind != Json::OBJ) return PB200_EINVAL;
    const ArchEntry * arch = arch_find(cfg.string("architecture").c_str());
    if (!arch || arch->family != ARCH_LAYERS) return PB200_ENOTSUP;
    pb200_model * m = pb200_model_create_from_config(cfg_text.c_str(), compute_type, device, n_ctx, n_seq);
    if (!m) return PB200_EINVAL;
    const int fd = open((d + "/model.safetensors").c_str(), O_RDONLY);
    if (fd < 0) { pb200_model_free(m); return PB200_EINVAL; }
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); pb200_model_free(m); return PB200_EINVAL; }
    const size_t fsz = (size_t) sb.st_size;
    void * map = mmap(nullptr, fsz, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) { pb200_model_free(m); return PB200_EINVAL; }
    const uint8_t * base = (const uint8_t *) map;
    int rc = 0;
    uint64_t hlen = 0;
    memcpy(&hlen, base, 8);
    Json hdr;
    if (hlen > fsz - 8 || !JsonParser((const char *) base + 8, (size_t) hlen).parse(hdr) || hdr.kind != Json::OBJ) rc = PB200_EINVAL;
    const uint8_t * data = base + 8 + hlen;
    const size_t dsz = fsz - 8 - (size_t) hlen;
    for (size_t i = 0; rc == 0 && i < hdr.obj.size(); i++) {
        const std::string & name = hdr.obj[i].first;
        const Json & t = hdr.obj[i].second;
        if (name == "__metadata__") continue;
        const std::string dt = t.string("dtype");
        const Json * offs = t.get("data_offsets");
        if (!offs || offs->kind != Json::ARR || offs->arr.size() != 2) { rc = PB200_EINVAL; break; }
        const uint64_t lo = (uint64_t) offs->arr[0].num, hi = (uint64_t) offs->arr[1].num;
        if (lo > hi || hi > dsz) { rc = PB200_EINVAL; break; }
        const int type = dt == "BF16" ? T_BF16 : dt == "F32" ? T_F32 : -1;
        TensorPlace pl;
        if (!m->ll->arch->resolve(*m->ll, name, pl)) {   // a tensor the design has no place for is left out; finalize still refuses an incomplete model
            fprintf(stderr, "[pb200] tensor '%s' is not part of %s: skipped\n", name.c_str(), arch->name);
            continue;
        }
        if (type < 0) { rc = PB200_ENOTSUP; fprintf(stderr, "[pb200] tensor '%s': dtype %s\n", name.c_str(), dt.c_str()); break; }
        rc = pb200_model_set_tensor(m, name.c_str(), type, data + lo, (size_t) (hi - lo));
        if (rc) fprintf(stderr, "[pb200] tensor '%s': %s\n", name.c_str(), pb200_error_string(rc));
    }
    munmap(map, fsz);
    if (rc == 0) rc = pb200_model_finalize(m);
    if (rc) { pb200_model_free(m); return rc; }
    *out = m;
    return 0;
}

int pb200_model_get_hparams(const pb200_model * m, pb200_hparams * out) {
    if (!m || !out) return PB200_EINVAL;
    *out = m->hp;
    return 0;
}
int pb200_model_n_seq(const pb200_model * m) { return m ? m->n_seq : 0; }

int pb200_seq_alloc(pb200_model * m) {
    if (!m) return PB200_EINVAL;
    if (!m->ll) return PB200_ENOTSUP;
    return ll_seq_alloc(m);
}
int pb200_seq_free(pb200_model * m, int slot) {
    if (!m) return PB200_EINVAL;
    if (!m->ll) return PB200_ENOTSUP;
    return ll_seq_free(m, slot);
}
int pb200_seq_length(pb200_model * m, int slot) {
    if (!m) return PB200_EINVAL;
    if (!m->ll) return PB200_ENOTSUP;
    return ll_seq_length(m, slot);
}
int pb200_batch_step(pb200_model * m, int n_entries, const pb200_batch_entry * entries, float * logits_host, int32_t * greedy_host) {
    if (!m) return PB200_EINVAL;
    if (!m->ll) return PB200_ENOTSUP;
    return ll_batch_step(m, n_entries, entries, logits_host, greedy_host);
}
int pb200_dense(int type, const void * A, int64_t lda, const void * W, int64_t ldw, float * C, int64_t ldc, int T, int N, int K, const float * bias,
                const float * resid, int64_t ldr, float alpha, void * stream) {
    if (type != T_F32 && type != T_BF16) return PB200_ENOTSUP;
    if (!A || !W || !C || T < 0 || N < 0 || K <= 0 || lda < K || ldw < K || ldc < N || (resid && ldr < N)) return PB200_EINVAL;
    return launch_dense(type, A, lda, W, ldw, C, ldc, T, N, K, bias, resid, ldr, alpha, (cudaStream_t) stream);
}
int pb200_debug_profile(pb200_model * m, int on) {
    if (!m || !m->ll) return PB200_EINVAL;
    m->ll->prof_on = on != 0;
    return 0;
}
int pb200_debug_tap_layers(pb200_model * m, int on) {
    if (!m || !m->ll) return PB200_EINVAL;
    m->ll->tap_on = on != 0;
    return 0;
}

}  // extern "C"
