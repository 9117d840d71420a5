// libwino C ABI: argument validation, problem geometry, slab scheduling and dispatch to the kernels.
//
// Host-side counterpart of the reference wrappers wrapedConv_NCHW / _NHWC / _CHWN
// (comparison/wrapedConv_NCHW.cuh:335-492, wrapedConv_NHWC.cuh:24-112, wrapedConv_CHWN.cuh:16-82):
// tiling arithmetic, then input transform -> tile GEMM -> output transform.  Differences by design:
//   * the filter transform is a separate call made once per weight tensor;
//   * the batch is processed in slabs of images that fit the caller's scratch (2 GiB by default, normally the
//     whole batch: slabs small enough to stay in the 126 MB L2 were measured and lose, their kernels are
//     launch- and latency-bound);
//   * thin and medium-width tensor-core layers leave the Winograd pipeline for a direct implicit-GEMM kernel
//     (direct_small_c.cu, direct_tc*.cu), chosen per shape and, for 512-channel layers, per batch size;
//   * everything is asynchronous on the caller's stream; only wino_wraped_conv synchronises.
#include <atomic>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "ptx.cuh"

namespace wino {

static thread_local char g_err[512] = "no error";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// ---- measurement hooks ---------------------------------------------------------------------------------
static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

namespace {
struct ProfRecord {
    cudaEvent_t start, stop;
    int stage;
};
std::mutex g_prof_mutex;
bool g_prof_on = false;
std::vector<ProfRecord> g_prof;
}  // namespace

ProfScope::ProfScope(int stage, cudaStream_t s) : slot(-1), st(s) {
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (!g_prof_on) return;
    ProfRecord r;
    r.stage = stage;
    if (cudaEventCreate(&r.start) != cudaSuccess) return;
    if (cudaEventCreate(&r.stop) != cudaSuccess) { cudaEventDestroy(r.start); return; }
    cudaEventRecord(r.start, st);
    g_prof.push_back(r);
    slot = (int)g_prof.size() - 1;
}

ProfScope::~ProfScope() {
    if (slot < 0) return;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (slot < (int)g_prof.size()) cudaEventRecord(g_prof[slot].stop, st);
}

static bool layout_ok(int l) { return l == WINO_NCHW || l == WINO_NHWC || l == WINO_CHWN; }

// Validates a descriptor and derives the tiling.  Mirrors wrapedConv_NCHW.cuh:346-362 (inside_beta,
// blockn, M/N/K sizes) with rectangular images and without the 128/128 padding of M and N.
int make_geometry(const wino_conv_desc* d, Geometry* g) {
    if (!d) return fail(WINO_E_BADARG, "descriptor is NULL");
    if (!layout_ok(d->layout_in) || !layout_ok(d->layout_out))
        return fail(WINO_E_BADARG, "bad layout code (in %d, out %d)", d->layout_in, d->layout_out);
    if (d->n < 0 || d->c <= 0 || d->h <= 0 || d->w <= 0 || d->k <= 0)
        return fail(WINO_E_BADARG, "bad shape n=%d c=%d h=%d w=%d k=%d", d->n, d->c, d->h, d->w, d->k);
    if (d->pad < 0 || d->pad > 1)
        return fail(WINO_E_UNSUPPORTED, "padding %d not supported (0 or 1; every reference caller passes 1)", d->pad);
    if (d->h + 2 * d->pad < 3 || d->w + 2 * d->pad < 3) return fail(WINO_E_BADARG, "image smaller than the 3x3 filter");
    if (d->wino != 0 && d->wino != 2 && d->wino != 4) return fail(WINO_E_BADARG, "wino must be 0, 2 or 4, got %d", d->wino);
    g->m = d->wino == 0 ? 4 : d->wino;
    g->a = g->m + 2;
    switch (d->dtype) {
        case WINO_FP32: g->operand = OP_F32; g->esize_io = 4; g->esize_op = 4; break;
        case WINO_TF32: g->operand = OP_TF32; g->esize_io = 4; g->esize_op = 4; break;
        case WINO_FP32X3: g->operand = OP_TF32X3; g->esize_io = 4; g->esize_op = 4; break;
        case WINO_BF16:
            g->esize_io = 2; g->esize_op = 2;
            if (d->operand == WINO_OPERAND_AUTO) g->operand = OP_F16;
            else if (d->operand == WINO_OPERAND_BF16) g->operand = OP_BF16;
            else if (d->operand == WINO_OPERAND_F16) g->operand = OP_F16;
            else return fail(WINO_E_BADARG, "bad operand code %d", d->operand);
            break;
        default: return fail(WINO_E_BADARG, "bad dtype code %d", d->dtype);
    }
    if (d->out_dtype != WINO_OUT_SAME && d->out_dtype != WINO_OUT_FP32 && d->out_dtype != WINO_OUT_BF16)
        return fail(WINO_E_BADARG, "bad out_dtype code %d", d->out_dtype);
    g->out_bf16 = d->out_dtype == WINO_OUT_SAME ? d->dtype == WINO_BF16 : d->out_dtype == WINO_OUT_BF16;
    g->oh = d->h + 2 * d->pad - 2;
    g->ow = d->w + 2 * d->pad - 2;
    if (d->pool2x2 && (g->oh < 2 || g->ow < 2)) return fail(WINO_E_BADARG, "pool2x2 needs an output of at least 2x2");
    g->ph = d->pool2x2 ? g->oh / 2 : g->oh;
    g->pw = d->pool2x2 ? g->ow / 2 : g->ow;
    g->bny = (g->oh + g->m - 1) / g->m;
    g->bnx = (g->ow + g->m - 1) / g->m;
    g->tiles_img = g->bny * g->bnx;
    g->cp = round_up(d->c, 8);
    g->crow = g->operand == OP_TF32X3 ? 2 * g->cp : g->cp;
    g->kq = round_up(d->k, 8);
    // What wino_conv_forward's tile GEMM writes.  The exact-FP32 path keeps the raw products M.  The tensor-core
    // paths write the row-transformed products Z (float for TF32, half for BF16 storage) when the layer is bound
    // by product traffic (C <= 128); for wider layers the tile GEMM is bound by filling shared memory with
    // operands and the 128-filter tiles of the plain kernel win.  WINO_ROWFUSE=0/1 forces either choice.
    {
        static const int force = [] { const char* e = getenv("WINO_ROWFUSE"); return e ? atoi(e) : -1; }();
        const bool fuse = g->operand != OP_F32 && g->operand != OP_TF32X3 && (force >= 0 ? force != 0 : d->c <= 128);
        g->prod_kind = !fuse ? 0 : g->operand == OP_TF32 ? 1 : 2;
    }
    g->prod_planes = g->prod_kind == 0 ? g->a * g->a : g->a * g->m;
    g->esize_prod = g->prod_kind == 2 ? 2 : 4;
    return WINO_OK;
}

static long long slab_budget_bytes() {
    static long long budget = [] {
        const char* e = getenv("WINO_SLAB_BYTES");
        long long v = e ? atoll(e) : 0;
        return v > 0 ? v : (2048LL << 20);
    }();
    return budget;
}

long long per_image_bytes(const Geometry& g) {
    return (long long)g.tiles_img * ((long long)g.a * g.a * g.cp * g.esize_op + (long long)g.prod_planes * g.kq * g.esize_prod);
}

// images per slab
static int slab_images(const wino_conv_desc& d, const Geometry& g) {
    if (d.n == 0) return 0;
    long long ns = d.slab_images > 0 ? d.slab_images : slab_budget_bytes() / per_image_bytes(g);
    if (ns < 1) ns = 1;
    if (ns > d.n) ns = d.n;
    if (ns > 65535) ns = 65535;
    // several slabs: start each on a multiple of 8 images, so that the CHWN kernels keep their 16-byte vectors along n
    if (ns < d.n && ns >= 8 && d.slab_images <= 0) ns -= ns % 8;
    return (int)ns;
}

long long tile_rows(const Geometry& g, int ns) { return round_up_ll((long long)ns * g.tiles_img, 128); }

size_t v_bytes(const Geometry& g, long long tp) {
    return (size_t)round_up_ll((long long)g.a * g.a * tp * g.cp * g.esize_op, 1024);
}
size_t m_bytes(const Geometry& g, long long tp) {
    return (size_t)round_up_ll((long long)g.a * g.a * tp * g.kq * 4, 1024);
}

size_t prod_bytes(const Geometry& g, long long tp) {
    return (size_t)round_up_ll((long long)g.prod_planes * tp * g.kq * g.esize_prod, 1024);
}

int run_gemm(const Geometry& g, const void* v, const void* u, float* m, int k, long long t_rows, long long tp,
                    cudaStream_t st) {
    if (g.operand == OP_F32)
        return launch_gemm_ffma((const float*)v, (const float*)u, m, g.a * g.a, t_rows, tp, k, g.cp, g.kq, st);
    if (g.operand == OP_TF32X3)
        return launch_gemm_tc_split((const float*)v, (const float*)u, m, g.a * g.a, t_rows, tp, k, g.cp, g.kq, st);
    return launch_gemm_tc(g.operand, v, u, m, g.a * g.a, t_rows, tp, k, g.cp, g.kq, st);
}

int run_conv_gemm(const Geometry& g, const void* v, const void* u, void* prod, int k, long long t_rows, long long tp,
                  cudaStream_t st) {
    if (g.prod_kind == 0) return run_gemm(g, v, u, (float*)prod, k, t_rows, tp, st);
    return launch_gemm_tc_z(g.operand, g.a, v, u, prod, t_rows, tp, k, g.cp, g.kq, st);
}

// stage-level entry points of the row-fused pair use Z whatever the layer width
static bool force_rowfused(Geometry* g) {
    if (g->operand == OP_F32 || g->operand == OP_TF32X3) return false;
    g->prod_kind = g->operand == OP_TF32 ? 1 : 2;
    g->prod_planes = g->a * g->m;
    g->esize_prod = g->prod_kind == 2 ? 2 : 4;
    return true;
}

// ---- filter buffer layout ------------------------------------------------------------------------------------
size_t wino_u_bytes(const wino_conv_desc& d, const Geometry& g) { return (size_t)g.a * g.a * d.k * g.crow * g.esize_op; }
// where the packed filters of the direct kernel start in a buffer that holds both forms (direct_filter_mode == 2)
size_t direct_filter_offset(const wino_conv_desc& d, const Geometry& g) { return (size_t)round_up_ll((long long)wino_u_bytes(d, g), 1024); }
const void* direct_filters(const wino_conv_desc& d, const Geometry& g, const void* u) {
    return direct_filter_mode(d) == 2 ? (const char*)u + direct_filter_offset(d, g) : u;
}

int check_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(WINO_E_CUDA, "no usable CUDA device: %s (libwino has no CPU path)", cudaGetErrorString(e));
    }
    return WINO_OK;
}

}  // namespace wino

using namespace wino;

extern "C" {

const char* wino_last_error_string(void) { return g_err; }

int wino_version(void) { return 100; }

long long wino_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int wino_profile_enable(int on) {
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof_on = on != 0;
    return WINO_OK;
}

int wino_profile_read(float stage_ms[8], long long stage_launches[8]) {
    if (!stage_ms || !stage_launches) return fail(WINO_E_BADARG, "profile read: NULL pointer");
    for (int i = 0; i < STAGE_COUNT; ++i) { stage_ms[i] = 0.f; stage_launches[i] = 0; }
    int rc = check_device();
    if (rc) return rc;
    WINO_CUDA_CHECK(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    for (ProfRecord& r : g_prof) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.start, r.stop) == cudaSuccess && r.stage >= 0 && r.stage < STAGE_COUNT) {
            stage_ms[r.stage] += ms;
            stage_launches[r.stage] += 1;
        }
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    g_prof.clear();
    return WINO_OK;
}

int wino_device_status(void) {
    int rc = check_device();
    if (rc) return rc;
    int s = 0;
    if ((rc = read_and_clear_status(&s))) return rc;
    if (s != 0) return fail(WINO_E_TIMEOUT, "a CTA gave up a bounded wait (code %d: tile GEMM 1 ring slot free, 2 ring slot filled, 3 accumulator drained, 4 accumulator ready; 5, 6 input-transform patch load; 1x row-fused GEMM, 2x CTA-pair GEMM, 4x direct convolution, 90 self-test)", s);
    return WINO_OK;
}

size_t wino_filter_bytes(const wino_conv_desc* d) {
    Geometry g;
    if (make_geometry(d, &g) != WINO_OK) return 0;
    if (direct_small_c_applies(*d)) {
        // thin-input layers keep packed raw filters (always smaller); report the larger so either kernel's buffer fits
        const size_t wino = wino_u_bytes(*d, g), thin = direct_small_c_filter_bytes(*d);
        return thin > wino ? thin : wino;
    }
    const int mode = direct_filter_mode(*d);
    if (mode == 1) { const size_t wino = wino_u_bytes(*d, g), dir = direct_tc_filter_bytes(*d); return dir > wino ? dir : wino; }
    if (mode == 2) return direct_filter_offset(*d, g) + direct_tc_filter_bytes(*d);
    return wino_u_bytes(*d, g);
}

size_t wino_conv_workspace_bytes(const wino_conv_desc* d) {
    Geometry g;
    if (make_geometry(d, &g) != WINO_OK) return 0;
    if (direct_via_nhwc_applies(*d)) return direct_via_nhwc_staging_bytes(*d, g);
    const long long tp = tile_rows(g, slab_images(*d, g));
    return v_bytes(g, tp) + prod_bytes(g, tp) + 1024;
}

long long wino_stage_tile_rows(const wino_conv_desc* d, int ns) {
    Geometry g;
    if (make_geometry(d, &g) != WINO_OK) return -1;
    return tile_rows(g, ns);
}

int wino_stage_cp(const wino_conv_desc* d) {
    Geometry g;
    if (make_geometry(d, &g) != WINO_OK) return -1;
    return g.cp;
}

int wino_stage_kq(const wino_conv_desc* d) {
    Geometry g;
    if (make_geometry(d, &g) != WINO_OK) return -1;
    return g.kq;
}

int wino_filter_transform(const wino_conv_desc* d, const void* w, void* u, wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (!w || !u) return fail(WINO_E_BADARG, "filter transform: NULL pointer");
    if ((rc = check_device())) return rc;
    if (direct_small_c_applies(*d)) return launch_direct_small_c_pack(*d, w, u, (cudaStream_t)stream);
    // The format of `u` depends on the shape, never on the batch size: where the engine picks between the direct kernel
    // and the Winograd pipeline by batch size, `u` holds both forms and forward calls of any batch size can share it.
    const int mode = direct_filter_mode(*d);
    if (mode == 1) return launch_direct_tc_pack(*d, w, u, (cudaStream_t)stream);
    if ((rc = launch_filter_transform(*d, g, w, u, (cudaStream_t)stream))) return rc;
    if (mode == 2) return launch_direct_tc_pack(*d, w, (char*)u + direct_filter_offset(*d, g), (cudaStream_t)stream);
    return WINO_OK;
}

int wino_stage_input_transform(const wino_conv_desc* d, const void* x, int n0, int ns, void* v, wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (!x || !v) return fail(WINO_E_BADARG, "input transform: NULL pointer");
    if (n0 < 0 || ns < 0 || n0 + ns > d->n) return fail(WINO_E_BADARG, "input transform: slab [%d, %d) outside batch %d", n0, n0 + ns, d->n);
    if ((rc = check_device())) return rc;
    return launch_input_transform(*d, g, x, n0, ns, v, tile_rows(g, ns), (cudaStream_t)stream);
}

int wino_stage_gemm(const wino_conv_desc* d, const void* v, const void* u, float* m, int ns, wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (!v || !u || !m) return fail(WINO_E_BADARG, "tile gemm: NULL pointer");
    if (ns < 0) return fail(WINO_E_BADARG, "tile gemm: negative slab");
    if ((rc = check_device())) return rc;
    return run_gemm(g, v, u, m, d->k, (long long)ns * g.tiles_img, tile_rows(g, ns), (cudaStream_t)stream);
}

int wino_stage_output_transform(const wino_conv_desc* d, const float* m, const float* bias, void* y, int n0, int ns,
                                wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (!m || !y) return fail(WINO_E_BADARG, "output transform: NULL pointer");
    if (d->has_bias && !bias) return fail(WINO_E_BADARG, "output transform: has_bias set but bias is NULL");
    if (n0 < 0 || ns < 0 || n0 + ns > d->n) return fail(WINO_E_BADARG, "output transform: slab [%d, %d) outside batch %d", n0, n0 + ns, d->n);
    if ((rc = check_device())) return rc;
    return launch_output_transform(*d, g, m, 0, bias, y, n0, ns, tile_rows(g, ns), (cudaStream_t)stream);
}

int wino_stage_gemm_rowfused(const wino_conv_desc* d, const void* v, const void* u, void* z, int ns, wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (!force_rowfused(&g)) return fail(WINO_E_UNSUPPORTED, "row-fused tile gemm exists for the tensor-core variants (TF32, BF16) only");
    if (!v || !u || !z) return fail(WINO_E_BADARG, "row-fused tile gemm: NULL pointer");
    if (ns < 0) return fail(WINO_E_BADARG, "row-fused tile gemm: negative slab");
    if ((rc = check_device())) return rc;
    return run_conv_gemm(g, v, u, z, d->k, (long long)ns * g.tiles_img, tile_rows(g, ns), (cudaStream_t)stream);
}

int wino_stage_output_transform_rowfused(const wino_conv_desc* d, const void* z, const float* bias, void* y, int n0, int ns,
                                         wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (!force_rowfused(&g)) return fail(WINO_E_UNSUPPORTED, "row-fused output transform exists for the tensor-core variants (TF32, BF16) only");
    if (!z || !y) return fail(WINO_E_BADARG, "row-fused output transform: NULL pointer");
    if (d->has_bias && !bias) return fail(WINO_E_BADARG, "row-fused output transform: has_bias set but bias is NULL");
    if (n0 < 0 || ns < 0 || n0 + ns > d->n) return fail(WINO_E_BADARG, "row-fused output transform: slab [%d, %d) outside batch %d", n0, n0 + ns, d->n);
    if ((rc = check_device())) return rc;
    return launch_output_transform(*d, g, z, g.prod_kind, bias, y, n0, ns, tile_rows(g, ns), (cudaStream_t)stream);
}

int wino_conv_forward(const wino_conv_desc* d, const void* x, const void* u, const float* bias, void* y,
                      void* workspace, size_t workspace_bytes, wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (d->n == 0) return WINO_OK;
    if (!x || !u || !y) return fail(WINO_E_BADARG, "conv forward: NULL tensor pointer");
    if (d->has_bias && !bias) return fail(WINO_E_BADARG, "conv forward: has_bias set but bias is NULL");
    if ((rc = check_device())) return rc;
    if (direct_small_c_applies(*d)) return launch_direct_small_c(*d, g, x, u, bias, y, (cudaStream_t)stream);
    if (direct_tc_applies(*d)) return launch_direct_tc(*d, g, x, direct_filters(*d, g, u), bias, y, (cudaStream_t)stream);
    if (direct_via_nhwc_applies(*d))
        return launch_direct_via_nhwc(*d, g, x, direct_filters(*d, g, u), bias, y, workspace, workspace_bytes, (cudaStream_t)stream);
    const int ns = slab_images(*d, g);
    const long long tp = tile_rows(g, ns);
    const size_t need = v_bytes(g, tp) + prod_bytes(g, tp) + 1024;
    if (!workspace || workspace_bytes < need)
        return fail(WINO_E_WORKSPACE, "conv forward: workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    // carve the workspace on 1 KiB boundaries
    uintptr_t base = ((uintptr_t)workspace + 1023) & ~(uintptr_t)1023;
    void* v = (void*)base;
    void* prod = (void*)(base + v_bytes(g, tp));
    cudaStream_t st = (cudaStream_t)stream;
    // Wide tensor-core layers with an NHWC result: the raw products cross HBM in 3 bytes instead of 4 (they fit the same
    // buffer).  Decided once per call from the whole batch, so that the result does not depend on the slab size; it
    // needs nothing from the filter buffer.
    const bool m24 = g.prod_kind == 0 && gemm_tc_m24_applies(g.operand, d->k, g.cp, g.kq, (long long)d->n * g.tiles_img) &&
                     output_transform_m24_ok(*d, y) && (long long)g.a * g.a * tp * g.kq * 2 < (1LL << 32);
    for (int n0 = 0; n0 < d->n; n0 += ns) {
        const int cur = d->n - n0 < ns ? d->n - n0 : ns;
        if ((rc = launch_input_transform(*d, g, x, n0, cur, v, tp, st))) return rc;
        const long long t_rows = (long long)cur * g.tiles_img;
        if (m24) {
            if ((rc = launch_gemm_tc_pair(g.operand, v, u, (float*)prod, g.a * g.a, t_rows, tp, d->k, g.cp, g.kq, st, true))) return rc;
            if ((rc = launch_output_transform(*d, g, prod, 3, bias, y, n0, cur, tp, st))) return rc;
            continue;
        }
        if ((rc = run_conv_gemm(g, v, u, prod, d->k, t_rows, tp, st))) return rc;
        if ((rc = launch_output_transform(*d, g, prod, g.prod_kind, bias, y, n0, cur, tp, st))) return rc;
    }
    return WINO_OK;
}

int wino_wraped_conv(int layout_src, int layout_dst, int bat4Conv, int inside, int* chn, int numOfFilter, int padding,
                     float* m1, float* m2, float* inputTran_gpu, float* filterTran_gpu, float* gemmOutput_gpu,
                     float** output) {
    if (!chn || !output || !*output) return fail(WINO_E_BADARG, "wraped conv: NULL chn/output");
    if (!inputTran_gpu || !filterTran_gpu || !gemmOutput_gpu) return fail(WINO_E_BADARG, "wraped conv: NULL workspace");
    wino_conv_desc d;
    memset(&d, 0, sizeof(d));
    d.layout_in = layout_src; d.layout_out = layout_dst;
    d.n = bat4Conv; d.c = *chn; d.h = inside; d.w = inside; d.k = numOfFilter; d.pad = padding;
    d.dtype = WINO_FP32; d.wino = 4;
    Geometry g;
    int rc = make_geometry(&d, &g);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    if (d.n > 0) {
        // Slabs are carved out of the caller's legacy buffers.  Their guaranteed minimum sizes
        // (36*Mp*Kp and 36*Mp*Np floats with Mp = roundup(N*bn*bn, 128), layoutTest/NCHW/convModule_NCHW_padding.cu:44-50)
        // cover V and M of the whole batch in this library's layouts, hence of any slab.
        const int ns = slab_images(d, g);
        const long long tp = tile_rows(g, ns);
        if ((rc = launch_filter_transform(d, g, m2, filterTran_gpu, 0))) return rc;
        for (int n0 = 0; n0 < d.n; n0 += ns) {
            const int cur = d.n - n0 < ns ? d.n - n0 : ns;
            if ((rc = launch_input_transform(d, g, m1, n0, cur, inputTran_gpu, tp, 0))) return rc;
            if ((rc = run_gemm(g, inputTran_gpu, filterTran_gpu, gemmOutput_gpu, d.k, (long long)cur * g.tiles_img, tp, 0))) return rc;
            if ((rc = launch_output_transform(d, g, gemmOutput_gpu, 0, nullptr, *output, n0, cur, tp, 0))) return rc;
        }
    }
    WINO_CUDA_CHECK(cudaDeviceSynchronize());  // the reference wrappers return synchronised (wrapedConv_NCHW.cuh:482)
    WINO_CUDA_CHECK(cudaGetLastError());
    *chn = numOfFilter;                        // wrapedConv_NCHW.cuh:479
    return WINO_OK;
}

int wino_layout_convert(int layout_src, int layout_dst, int n, int c, int h, int w, int dtype, const void* in, void* out,
                        wino_stream_t stream) {
    if (!layout_ok(layout_src) || !layout_ok(layout_dst)) return fail(WINO_E_BADARG, "layout convert: bad layout code");
    if (n < 0 || c < 0 || h < 0 || w < 0) return fail(WINO_E_BADARG, "layout convert: negative extent");
    if (dtype != WINO_FP32 && dtype != WINO_TF32 && dtype != WINO_BF16 && dtype != WINO_FP32X3) return fail(WINO_E_BADARG, "layout convert: bad dtype %d", dtype);
    if ((long long)n * c * h * w == 0) return WINO_OK;
    if (!in || !out) return fail(WINO_E_BADARG, "layout convert: NULL pointer");
    int rc = check_device();
    if (rc) return rc;
    return launch_relayout(layout_src, layout_dst, n, c, h, w, dtype == WINO_BF16 ? 2 : 4, in, out, (cudaStream_t)stream);
}

int wino_maxpool2x2(int layout, int n, int c, int h, int w, int dtype, const void* in, void* out, wino_stream_t stream) {
    if (!layout_ok(layout)) return fail(WINO_E_BADARG, "maxpool: bad layout code");
    if (n < 0 || c < 0 || h < 0 || w < 0) return fail(WINO_E_BADARG, "maxpool: negative extent");
    if (dtype != WINO_FP32 && dtype != WINO_TF32 && dtype != WINO_BF16 && dtype != WINO_FP32X3) return fail(WINO_E_BADARG, "maxpool: bad dtype %d", dtype);
    if ((long long)n * c * (h / 2) * (w / 2) == 0) return WINO_OK;
    if (!in || !out) return fail(WINO_E_BADARG, "maxpool: NULL pointer");
    int rc = check_device();
    if (rc) return rc;
    return launch_maxpool(layout, n, c, h, w, dtype, in, out, (cudaStream_t)stream);
}

}  // extern "C"
