// extern "C" entry points of libgeo_sc.so and the host-side geometry / planning logic.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "sc_common.h"
#include "sc_fullbin.h"
#include "sc_guide_tc.h"
#include "sc_rows.h"
#include "sc_short.h"
#include "sc_sorted.h"
#include "sc_taps.h"

namespace geo {

static thread_local char g_err[512] = "";

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

int sm_count() {
    static std::mutex m;
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(m);
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static int lfsr_bits(int L) {
    switch (L) {
    case 8: return 3;
    case 16: return 4;
    case 32: return 5;
    case 64: return 6;
    case 128: return 7;
    case 256: return 8;
    default: return 0;
    }
}

int make_geometry(const geo_sc_conv_desc *d, Geometry *g) {
    if (!d || !g) return fail(GEO_SC_ERR_NULL, "descriptor is NULL");
    memset(g, 0, sizeof(*g));
    g->nbits = lfsr_bits(d->bit_length);
    if (!g->nbits)
        return fail(GEO_SC_ERR_BIT_LENGTH, "bit_length %d is not one of 8,16,32,64,128,256", d->bit_length);
    if (d->mode < GEO_SC_MODE_1D || d->mode > GEO_SC_MODE_FULL_BIN) return fail(GEO_SC_ERR_MODE, "mode %d", d->mode);
    if (d->batch < 1 || d->c_in < 1 || d->h_in < 1 || d->w_in < 1 || d->c_out < 1 || d->k_h < 1 || d->k_w < 1 ||
        d->pad_h < 0 || d->pad_w < 0)
        return fail(GEO_SC_ERR_SHAPE, "non-positive dimension (batch %d c_in %d h %d w %d c_out %d k %dx%d pad %d,%d)",
                    d->batch, d->c_in, d->h_in, d->w_in, d->c_out, d->k_h, d->k_w, d->pad_h, d->pad_w);
    if (d->total_width < 0 || d->total_width > 15 || d->load_width < 1 || d->load_wait_w < 1 || d->load_wait_a < 1)
        return fail(GEO_SC_ERR_LOADING, "total_width %d load_width %d load_wait %d/%d (need 0<=tw<=15, others >=1)",
                    d->total_width, d->load_width, d->load_wait_w, d->load_wait_a);
    g->B = d->batch; g->C = d->c_in; g->H = d->h_in; g->W = d->w_in;
    g->pad_h = d->pad_h; g->pad_w = d->pad_w;
    long long Hp = (long long)d->h_in + 2LL * d->pad_h, Wp = (long long)d->w_in + 2LL * d->pad_w;
    if (Hp < d->k_h || Wp < d->k_w)
        return fail(GEO_SC_ERR_SHAPE, "filter %dx%d larger than padded image %lldx%lld", d->k_h, d->k_w, Hp, Wp);
    if (Hp > (1 << 20) || Wp > (1 << 20)) return fail(GEO_SC_ERR_TOO_LARGE, "padded image %lldx%lld", Hp, Wp);
    g->Hp = (int)Hp; g->Wp = (int)Wp;
    g->O = d->c_out; g->K2 = d->k_h; g->K3 = d->k_w;
    g->Ho = g->Hp - g->K2 + 1; g->Wo = g->Wp - g->K3 + 1;
    g->L = d->bit_length; g->P = (g->L + 31) / 32;
    g->mode = d->mode;
    g->guide_linear = 0;
    g->Bp = (d->batch + 3) / 4 * 4;
    g->batch_fast = 0;   // decided below, once the group geometry is known
    if (d->generator < GEO_SC_GEN_LFSR || d->generator > GEO_SC_GEN_RAND) return fail(GEO_SC_ERR_MODE, "generator %d", d->generator);
    g->generator = d->generator;
    g->seed = d->seed;
    g->tw = d->total_width; g->lu = d->load_width; g->lw_w = d->load_wait_w; g->lw_a = d->load_wait_a;
    g->z = 1;
    long long G, K;
    switch (g->mode) {
    case GEO_SC_MODE_1D: G = g->K3; K = (long long)g->C * g->K2; break;
    case GEO_SC_MODE_Z: G = g->C; K = (long long)g->K2 * g->K3; break;
    case GEO_SC_MODE_YZ:
        if (d->z_unit < 1) return fail(GEO_SC_ERR_SHAPE, "z_unit %d < 1", d->z_unit);
        g->z = d->z_unit < g->C ? d->z_unit : g->C;
        G = (long long)((g->C + g->z - 1) / g->z) * g->K3;
        K = (long long)g->z * g->K2;
        break;
    case GEO_SC_MODE_2D: G = (long long)g->K2 * g->K3; K = g->C; break;
    case GEO_SC_MODE_FULL_BIN: G = (long long)g->C * g->K2 * g->K3; K = 1; break;
    default: G = 1; K = (long long)g->C * g->K2 * g->K3; break;
    }
    g->NT = g->O <= 16 ? 16 : (g->O <= 32 ? 32 : 64);
    g->Opad = (g->O + g->NT - 1) / g->NT * g->NT;
    const long long lim = (1LL << 31) - 1;
    long long M = (long long)g->B * g->Ho * g->Wo;
    long long aw = (long long)g->Bp * g->P * g->C * g->Hp * g->Wp;   // bound for either layout
    // members as laid out: short groups are padded to a multiple of 4 (one stage holds the whole
    // group), longer ones to a multiple of 16 (stages of 16 or 32 members)
    const long long Kp = K <= 16 ? (K + 3) / 4 * 4 : (K + 15) / 16 * 16;
    long long ww = (long long)g->P * G * Kp * g->Opad * 2;
    long long ow = M * g->O;
    long long iw = (long long)g->B * g->C * g->H * g->W;
    if (G > lim || Kp > lim || M > lim || aw > lim || ww > lim || ow > lim || iw > lim || G * Kp > lim)
        return fail(GEO_SC_ERR_TOO_LARGE,
                    "an index exceeds 31 bits (positions %lld, act words %lld, weight words %lld, outputs %lld)", M, aw,
                    ww, ow);
    g->G = (int)G; g->K = (int)K; g->Kp = (int)Kp; g->M = M;
    g->w_stream_words = (size_t)ww;
    g->aoff_entries = (size_t)(G * Kp);
    // batch-innermost stream image: linear layers and the layers of the tap-tile kernel
    g->batch_fast = (g->Hp * g->Wp == 1 || taps_plan(*g).layout) ? 1 : 0;
    g->act_stream_words = (size_t)(g->batch_fast ? g->Bp : g->B) * g->P * g->C * g->Hp * g->Wp;
    return GEO_SC_OK;
}

void make_load_plan(int L, int tw, int lu, int lw, LoadPlan *plan) {
    memset(plan, 0, sizeof(*plan));
    int level_of_shift[32];
    for (int i = 0; i < 32; i++) level_of_shift[i] = -1;
    for (int t = 1; t <= L; t++) {
        long long cw = ((long long)(t / lw) + 1) * lu - 1;
        if (cw > tw) cw = tw;
        int sh = tw - (int)cw;
        if (level_of_shift[sh] < 0) {
            level_of_shift[sh] = plan->nlev;
            plan->shift[plan->nlev++] = sh;
        }
        int lev = level_of_shift[sh];
        int p, bit;
        if (L >= 32) { p = (t - 1) / 32; bit = 31 - (t - 1) % 32; }
        else { p = 0; bit = L - t; }
        plan->mask[p][lev] |= 1u << bit;
    }
    for (int p = 0; p < kMaxPacks; p++)
        for (int j = 0; j < plan->nlev; j++)
            if (plan->mask[p][j]) plan->act[p][plan->nact[p]++] = (unsigned char)j;
}

static size_t wprep_dense_bytes(const Geometry &g) {
    return align_up(g.w_stream_words * 4, 256) + align_up(g.aoff_entries * 4, 256);
}
// dense streams, member offsets, then one section for the kernel that applies one logic op per weight: for long
// groups the sign-sorted lists (the row-tile form where the layer's geometry allows it, else the im2col form), for
// short groups the per-chunk sorted lists of sc_accumulate_short.cu
static size_t wprep_bytes(const Geometry &g) {
    const FullBinPlan fb = fullbin_plan(g);
    if (fb.layout) return wprep_dense_bytes(g) + fb.bytes;   // full_bin: the weights packed for the binary GEMM
    const TapsPlan tp = taps_plan(g);
    if (tp.layout) return wprep_dense_bytes(g) + tp.total();
    const RowsPlan rp = rows_plan(g);
    if (rp.layout) return wprep_dense_bytes(g) + rp.total();
    const SortedPlan so = sorted_plan(g);
    return wprep_dense_bytes(g) + (so.layout ? so.total() : short_plan(g).total());
}

static int prepare_all(const Geometry &g, const float *weight, void *wprep, cudaStream_t s) {
    uint32_t *ws = (uint32_t *)wprep;
    int32_t *aoff = (int32_t *)((char *)wprep + align_up(g.w_stream_words * 4, 256));
    int rc = launch_prepare_weights(g, weight, ws, aoff, s);
    if (rc) return rc;
    if (fullbin_plan(g).layout) rc = launch_fullbin_pack(g, ws, (char *)wprep + wprep_dense_bytes(g), s);
    else if (taps_plan(g).layout) rc = launch_sort_taps(g, ws, (char *)wprep + wprep_dense_bytes(g), s);
    else if (rows_plan(g).layout) rc = launch_sort_rows(g, ws, (char *)wprep + wprep_dense_bytes(g), s);
    else if (sorted_plan(g).layout) rc = launch_sort_members(g, ws, (char *)wprep + wprep_dense_bytes(g), s);
    else if (short_plan(g).layout) rc = launch_sort_short(g, ws, (char *)wprep + wprep_dense_bytes(g), s);
    return rc;
}

// which kernel a launch gets (GEO_SC_KERNEL_*): the one place that decides
static int accumulate_kernel_of(const Geometry &g) {
    if (fullbin_plan(g).layout) return GEO_SC_KERNEL_FULL_BIN;
    const TapsPlan tp = taps_plan(g);
    if (tp.layout) return tp.eligible ? GEO_SC_KERNEL_SORTED_TAPS : GEO_SC_KERNEL_DENSE;
    const RowsPlan rp = rows_plan(g);
    if (rp.eligible) return GEO_SC_KERNEL_SORTED_ROWS;
    if (rp.layout) return GEO_SC_KERNEL_DENSE;   // the row-tile section is the only sorted one in the buffer
    const SortedPlan so = sorted_plan(g);
    if (so.eligible) return GEO_SC_KERNEL_SORTED_IM2COL;
    if (so.layout) return GEO_SC_KERNEL_DENSE;
    return short_plan(g).eligible ? GEO_SC_KERNEL_SORTED_SHORT : GEO_SC_KERNEL_DENSE;
}

static int accumulate_any(const Geometry &g, const uint32_t *as, const void *wprep, int32_t *out, cudaStream_t s) {
    const uint32_t *ws = (const uint32_t *)wprep;
    const int32_t *aoff = (const int32_t *)((const char *)wprep + align_up(g.w_stream_words * 4, 256));
    const void *section = (const char *)wprep + wprep_dense_bytes(g);
    switch (accumulate_kernel_of(g)) {
    case GEO_SC_KERNEL_FULL_BIN: return launch_accumulate_fullbin(g, as, aoff, section, out, s);
    case GEO_SC_KERNEL_SORTED_TAPS: return launch_accumulate_taps(g, as, section, out, s);
    case GEO_SC_KERNEL_SORTED_ROWS: return launch_accumulate_rows(g, as, section, out, s);
    case GEO_SC_KERNEL_SORTED_IM2COL: return launch_accumulate_sorted(g, as, aoff, section, out, s);
    case GEO_SC_KERNEL_SORTED_SHORT: return launch_accumulate_short(g, as, aoff, section, out, s);
    default: return launch_accumulate(g, as, ws, aoff, out, s);
    }
}
static size_t astream_bytes(const Geometry &g) { return align_up(g.act_stream_words * 4, 256); }

static int check_buffer(const void *p, size_t have, size_t need, const char *what) {
    if (!p) return fail(GEO_SC_ERR_NULL, "%s is NULL", what);
    if (((uintptr_t)p & 255) != 0) return fail(GEO_SC_ERR_WORKSPACE, "%s is not 256-byte aligned", what);
    if (have < need) return fail(GEO_SC_ERR_WORKSPACE, "%s holds %zu bytes, %zu needed", what, have, need);
    return GEO_SC_OK;
}

}  // namespace geo

using namespace geo;

extern "C" {

int geo_sc_version(void) { return GEO_SC_VERSION; }

const char *geo_sc_status_string(int status) {
    switch (status) {
    case GEO_SC_OK: return "ok";
    case GEO_SC_ERR_NULL: return "null pointer";
    case GEO_SC_ERR_BIT_LENGTH: return "unsupported bit_length";
    case GEO_SC_ERR_SHAPE: return "bad shape";
    case GEO_SC_ERR_MODE: return "unknown mode";
    case GEO_SC_ERR_LOADING: return "bad progressive-loading parameters";
    case GEO_SC_ERR_TOO_LARGE: return "problem too large for 31-bit indexing";
    case GEO_SC_ERR_WORKSPACE: return "workspace too small or misaligned";
    case GEO_SC_ERR_CUDA: return "CUDA runtime error";
    case GEO_SC_ERR_UNSUPPORTED: return "unsupported";
    default: return "unknown status";
    }
}

const char *geo_sc_last_error(void) { return g_err; }

int geo_sc_init(void) { return ensure_tables(); }

int geo_sc_device_error_count(int *count) {
    if (!count) return fail(GEO_SC_ERR_NULL, "count is NULL");
    return tc_error_count(count);
}

int geo_sc_group_geometry(const geo_sc_conv_desc *desc, int32_t *groups, int32_t *members, int32_t *members_padded,
                          int32_t *cout_tile, int32_t *cout_padded) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (groups) *groups = g.G;
    if (members) *members = g.K;
    if (members_padded) *members_padded = g.Kp;
    if (cout_tile) *cout_tile = g.NT;
    if (cout_padded) *cout_padded = g.Opad;
    return GEO_SC_OK;
}

int geo_sc_accumulate_is_sign_sorted(const geo_sc_conv_desc *desc, int *yes) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!yes) return fail(GEO_SC_ERR_NULL, "yes is NULL");
    const int k = accumulate_kernel_of(g);
    *yes = k == GEO_SC_KERNEL_SORTED_ROWS || k == GEO_SC_KERNEL_SORTED_IM2COL || k == GEO_SC_KERNEL_SORTED_SHORT ||
                   k == GEO_SC_KERNEL_SORTED_TAPS
               ? 1
               : 0;
    return GEO_SC_OK;
}

int geo_sc_accumulate_kernel(const geo_sc_conv_desc *desc, int *kernel) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!kernel) return fail(GEO_SC_ERR_NULL, "kernel is NULL");
    *kernel = accumulate_kernel_of(g);
    return GEO_SC_OK;
}

int geo_sc_weight_prep_bytes(const geo_sc_conv_desc *desc, size_t *bytes) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!bytes) return fail(GEO_SC_ERR_NULL, "bytes is NULL");
    *bytes = wprep_bytes(g);
    return GEO_SC_OK;
}

int geo_sc_act_stream_bytes(const geo_sc_conv_desc *desc, size_t *bytes) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!bytes) return fail(GEO_SC_ERR_NULL, "bytes is NULL");
    *bytes = astream_bytes(g);
    return GEO_SC_OK;
}

int geo_sc_act_stream_layout(const geo_sc_conv_desc *desc, int *batch_innermost, int *batch_padded) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (batch_innermost) *batch_innermost = g.batch_fast;
    if (batch_padded) *batch_padded = g.batch_fast ? g.Bp : g.B;
    return GEO_SC_OK;
}

int geo_sc_conv2d_workspace_bytes(const geo_sc_conv_desc *desc, size_t *bytes) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!bytes) return fail(GEO_SC_ERR_NULL, "bytes is NULL");
    *bytes = astream_bytes(g) + wprep_bytes(g);
    return GEO_SC_OK;
}

int geo_sc_prepare_weights(const geo_sc_conv_desc *desc, const float *weight, void *wprep, size_t bytes, void *stream) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!weight) return fail(GEO_SC_ERR_NULL, "weight is NULL");
    if ((rc = check_buffer(wprep, bytes, wprep_bytes(g), "prepared-weight buffer"))) return rc;
    return prepare_all(g, weight, wprep, (cudaStream_t)stream);
}

int geo_sc_generate_act_streams(const geo_sc_conv_desc *desc, const float *act, void *astream, size_t bytes,
                                void *stream) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!act) return fail(GEO_SC_ERR_NULL, "act is NULL");
    if ((rc = check_buffer(astream, bytes, astream_bytes(g), "activation-stream buffer"))) return rc;
    return launch_act_streams(g, act, (uint32_t *)astream, (cudaStream_t)stream);
}

int geo_sc_accumulate(const geo_sc_conv_desc *desc, const void *astream, const void *wprep, int32_t *out,
                      void *stream) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!astream || !wprep || !out) return fail(GEO_SC_ERR_NULL, "astream, wprep or out is NULL");
    if (((uintptr_t)astream & 15) || ((uintptr_t)wprep & 255))
        return fail(GEO_SC_ERR_WORKSPACE, "stream buffers are misaligned");
    return accumulate_any(g, (const uint32_t *)astream, wprep, out, (cudaStream_t)stream);
}

int geo_sc_conv2d_forward(const geo_sc_conv_desc *desc, const float *act, const float *weight, int32_t *out,
                          void *workspace, size_t workspace_bytes, void *stream) {
    Geometry g;
    int rc = make_geometry(desc, &g);
    if (rc) return rc;
    if (!act || !weight || !out) return fail(GEO_SC_ERR_NULL, "act, weight or out is NULL");
    size_t ab = astream_bytes(g), wb = wprep_bytes(g);
    if ((rc = check_buffer(workspace, workspace_bytes, ab + wb, "workspace"))) return rc;
    uint32_t *as = (uint32_t *)workspace;
    void *wprep = (char *)workspace + ab;
    cudaStream_t s = (cudaStream_t)stream;
    if ((rc = prepare_all(g, weight, wprep, s))) return rc;
    if ((rc = launch_act_streams(g, act, as, s))) return rc;
    return accumulate_any(g, as, wprep, out, s);
}

int geo_sc_linear_forward(const geo_sc_conv_desc *desc, const float *act, const float *weight, int32_t *out,
                          void *workspace, size_t workspace_bytes, void *stream) {
    if (!desc) return fail(GEO_SC_ERR_NULL, "descriptor is NULL");
    if (desc->h_in != 1 || desc->w_in != 1 || desc->k_h != 1 || desc->k_w != 1 || desc->pad_h || desc->pad_w)
        return fail(GEO_SC_ERR_SHAPE, "linear layer needs h_in=w_in=k_h=k_w=1 and no padding");
    geo_sc_conv_desc d = *desc;
    d.mode = GEO_SC_MODE_YZ;
    return geo_sc_conv2d_forward(&d, act, weight, out, workspace, workspace_bytes, stream);
}

}  // extern "C"
