// C ABI of the MoE layer: layer lifetime, parameter binding, workspace layout
// and the forward / backward schedules.  See include/mgpt_moe.h for the
// contract and the reference interfaces each entry point stands in for.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace mgpt {

static thread_local std::string g_error;
static std::atomic<long> g_launches{0};

void set_error(const std::string& msg) { g_error = msg; }
int fail(int code, const std::string& msg)
{
    g_error = msg;
    return code;
}
int cuda_fail(cudaError_t e, const char* what)
{
    g_error = std::string(what) + ": " + cudaGetErrorString(e);
    return MGPT_MOE_ECUDA;
}
void count_launch(int n) { g_launches += n; }

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

Workspace make_workspace(const Dims& d, int n_tokens, int kind)
{
    Workspace w = {};
    const size_t N = (size_t)n_tokens, E = d.E, k = d.k, C = d.C, H = d.H;
    w.n_tokens = n_tokens;
    w.R = (int)(N * k);
    w.max_tiles = (int)((N * k + E * (ROW_TILE - 1)) / ROW_TILE);
    if (w.max_tiles < 1) w.max_tiles = 1;
    w.row_cap = w.max_tiles * ROW_TILE;
    w.plan_blocks = (int)((N * k + 1023) / 1024);
    if (w.plan_blocks < 1) w.plan_blocks = 1;
    w.act_bytes = d.mode == MGPT_MOE_BF16 ? 2 : 4;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off = align_up(off + (bytes ? bytes : 1), 256);
        return o;
    };
    const size_t rc = (size_t)w.row_cap, ab = w.act_bytes;
    const size_t big = kind == 1 ? 0 : 1;          // routing-side workspaces carry no activation buffers
    const size_t rowbuf = (kind == 0 || kind == 3) ? 1 : 0;       // expert-side row buffers belong to the caller
    const size_t bwd = kind == 3 ? 0 : 1;          // inference keeps nothing for backward
    w.inference = kind == 3;
    w.logits = take(N * E * 4);
    w.probs = take(N * E * 4);
    w.top_idx = take(N * k * 4);
    w.top_p = take(N * k * 4);
    w.counts = take(E * 4);
    w.offsets = take(E * 4);
    w.padded_offsets = take((E + 1) * 4);
    w.tile_expert = take((size_t)w.max_tiles * 4);
    w.n_tiles = take(4);
    w.status = take(4);
    w.map = take(N * k * 4);
    w.pos = take(N * k * 4);
    w.row_src = take(rc * 4);
    w.pairs = take((size_t)w.max_tiles * 8);           // part of the plan: inside the range save_routing copies
    w.n_pairs = take(4);
    w.blk_cnt = take((size_t)w.plan_blocks * E * 4);
    w.slot = take(N * k * 4);
    w.seg = take(E * MAX_SOURCES * 2 * 4);
    w.tile_order = take((size_t)w.max_tiles * 4);
    w.Xg = take(rowbuf * rc * C * ab);
    w.G = take(bwd * big * rc * H * ab);
    w.U = take(bwd * big * rc * H * ab);
    w.Hh = take(big * rc * H * ab);
    w.Yg = take(rowbuf * rc * C * ab);
    w.dYg = take(bwd * rowbuf * rc * C * ab);
    w.dG = take(bwd * big * rc * H * ab);
    w.dU = take(bwd * big * rc * H * ab);
    w.dXg = take(bwd * rowbuf * rc * C * ab);
    w.d_top_p = take(bwd * N * k * 4);
    w.dlogits = take(bwd * N * E * 4);
    // router weight gradient: per-token-chunk partial sums, reduced in a second pass
    {
        const int e4 = (d.E + 3) / 4, ch_per_cta = (256 / e4) * 4;
        const int cblocks = (d.C + ch_per_cta - 1) / ch_per_cta;
        int chunks = 1184 / (cblocks > 0 ? cblocks : 1);
        if (chunks > 64) chunks = 64;
        if (chunks > n_tokens) chunks = n_tokens;
        if (chunks < 1) chunks = 1;
        w.rw_chunks = chunks;
    }
    w.rw_part = take(bwd * (size_t)w.rw_chunks * (C * E + E) * 4);
    w.dl16 = take(bwd * N * ((E + 7) / 8 * 8) * 2);          // dlogits in bf16 for the tensor-core router backward
    w.rt_list = take(N * 4);                            // screened router: tokens recomputed by the exact pass
    w.rt_count = take(4);
    w.total = off;
    return w;
}

static bool use_tc(const mgpt_moe_layer* L) { return L->d.mode == MGPT_MOE_BF16 && L->d.gemm_impl == 0; }

}  // namespace mgpt

using namespace mgpt;

extern "C" {

const char* mgpt_moe_last_error(void) { return g_error.c_str(); }

long mgpt_moe_launch_count(int reset)
{
    return reset ? g_launches.exchange(0) : g_launches.load();
}

int mgpt_moe_create(const mgpt_moe_config* cfg, mgpt_moe_layer** out)
{
    if (!cfg || !out) return fail(MGPT_MOE_EINVAL, "null argument");
    const int C = cfg->embed_dim, E = cfg->num_experts, k = cfg->top_k;
    const int H = cfg->hidden_dim == -1 ? 4 * C : cfg->hidden_dim;
    if (C <= 0 || H <= 0 || E <= 0 || k <= 0) return fail(MGPT_MOE_EINVAL, "dimensions must be positive");
    if (E > MAX_EXPERTS) return fail(MGPT_MOE_EINVAL, "num_experts > 128 is not supported");
    if (k > MAX_TOPK || k > E) return fail(MGPT_MOE_EINVAL, "top_k must be <= min(8, num_experts)");
    if (C % 8 || H % 8) return fail(MGPT_MOE_EINVAL, "embed_dim and hidden_dim must be multiples of 8");
    if (cfg->mode != MGPT_MOE_FP32 && cfg->mode != MGPT_MOE_BF16) return fail(MGPT_MOE_EINVAL, "unknown mode");
    int ndev = 0;
    MGPT_CUDA(cudaGetDeviceCount(&ndev));
    if (cfg->device < 0 || cfg->device >= ndev) return fail(MGPT_MOE_ECUDA, "no such CUDA device");
    MGPT_CUDA(cudaSetDevice(cfg->device));

    mgpt_moe_layer* L = new mgpt_moe_layer();
    L->d = Dims{C, H, E, k, cfg->lb_alpha, cfg->mode, cfg->gemm_impl};
    L->device = cfg->device;
    L->n_params = 2 + 6 * E;
    L->p_data.assign(L->n_params, nullptr);
    L->p_grad.assign(L->n_params, nullptr);

    // 15 tables of E pointers: 12 master (W, b, gW, gb) + 3 shadow W
    cudaError_t e = cudaMalloc(&L->d_tables, (size_t)15 * E * sizeof(void*));
    if (e != cudaSuccess) {
        delete L;
        return cuda_fail(e, "cudaMalloc(tables)");
    }
    void** t = (void**)L->d_tables;
    auto tab = [&](int i) { return t + (size_t)i * E; };
    L->master.Wg = (const void**)tab(0); L->master.Wu = (const void**)tab(1); L->master.Wd = (const void**)tab(2);
    L->master.bg = (const float**)tab(3); L->master.bu = (const float**)tab(4); L->master.bd = (const float**)tab(5);
    L->master.gWg = (float**)tab(6); L->master.gWu = (float**)tab(7); L->master.gWd = (float**)tab(8);
    L->master.gbg = (float**)tab(9); L->master.gbu = (float**)tab(10); L->master.gbd = (float**)tab(11);
    L->shadow = L->master;
    L->shadow.Wg = (const void**)tab(12); L->shadow.Wu = (const void**)tab(13); L->shadow.Wd = (const void**)tab(14);

    // error word of the layer's kernels (zero until something goes wrong) and the pinned word it is read into
    e = cudaMalloc(&L->d_status, 256);
    if (e == cudaSuccess) e = cudaMemset(L->d_status, 0, 256);
    if (e == cudaSuccess) e = cudaHostAlloc(&L->h_status, sizeof(int32_t), cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        mgpt_moe_destroy(L);
        return cuda_fail(e, "cudaMalloc(status)");
    }
    *L->h_status = 0;
    if (cfg->mode == MGPT_MOE_BF16 && cfg->gemm_impl == 0) {
        const int rc = tc_init(L);      // kernel attributes and the zeroed work-item counters, before any launch
        if (rc != 0) {
            mgpt_moe_destroy(L);
            return rc;
        }
    }
    if (cfg->mode == MGPT_MOE_BF16) {
        e = cudaMalloc(&L->sWr, (size_t)C * ((E + 7) / 8 * 8) * sizeof(bf16));
        if (e != cudaSuccess) {
            mgpt_moe_destroy(L);
            return cuda_fail(e, "cudaMalloc(router shadow)");
        }
        if (cfg->gemm_impl == 0) {
            if (const char* env = getenv("MGPT_MOE_ROUTER_TC_MIN_WORK")) L->router_tc_min_work = atof(env);
            L->router_ne = router_tc_ne(E);
            const size_t pieces = (size_t)2 * L->router_ne * C * sizeof(bf16);
            e = cudaMalloc(&L->sWrT2, pieces);
            if (e == cudaSuccess) e = cudaMemset(L->sWrT2, 0, pieces);      // rows of experts beyond E stay zero
            if (e == cudaSuccess) e = cudaMalloc(&L->d_rstat, 2 * sizeof(float));
            if (e == cudaSuccess) e = cudaMemset(L->d_rstat, 0, 2 * sizeof(float));
            if (e == cudaSuccess) e = cudaDeviceSynchronize();
            if (e != cudaSuccess) {
                mgpt_moe_destroy(L);
                return cuda_fail(e, "cudaMalloc(router pieces)");
            }
        }
        const size_t n = (size_t)E * C * H;
        bf16** s[6] = {&L->sWg, &L->sWu, &L->sWd, &L->sWgT, &L->sWuT, &L->sWdT};
        // the transposed copies are tile-major with zero padding up to whole 128 x 64 blocks
        const size_t ns[6] = {n, n, n, E * tile_major_elems(H, C), E * tile_major_elems(H, C), E * tile_major_elems(C, H)};
        for (int i = 0; i < 6; ++i) {
            e = cudaMalloc(s[i], ns[i] * sizeof(bf16));
            if (e == cudaSuccess && i >= 3) e = cudaMemset(*s[i], 0, ns[i] * sizeof(bf16));
            if (e != cudaSuccess) {
                mgpt_moe_destroy(L);
                return cuda_fail(e, "cudaMalloc(shadows)");
            }
        }
        e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            mgpt_moe_destroy(L);
            return cuda_fail(e, "clearing the weight copies");
        }
    }
    *out = L;
    return 0;
}

void mgpt_moe_destroy(mgpt_moe_layer* L)
{
    if (!L) return;
    cudaSetDevice(L->device);
    tc_destroy(L);
    cudaFree(L->d_tables);
    cudaFree(L->d_opt);
    cudaFree(L->d_status);
    if (L->h_status) cudaFreeHost(L->h_status);
    cudaFree(L->sWg); cudaFree(L->sWu); cudaFree(L->sWd);
    cudaFree(L->sWgT); cudaFree(L->sWuT); cudaFree(L->sWdT);
    cudaFree(L->sWr);
    cudaFree(L->sWrT2);
    cudaFree(L->d_rstat);
    cudaFree(L->h_x); cudaFree(L->h_dy); cudaFree(L->h_y); cudaFree(L->h_dx); cudaFree(L->h_ws);
    for (int s = 0; s < ST_COUNT; ++s) {
        if (L->ev_begin[s]) cudaEventDestroy(L->ev_begin[s]);
        if (L->ev_end[s]) cudaEventDestroy(L->ev_end[s]);
    }
    if (L->copy_stream) {
        cudaStreamDestroy(L->copy_stream);
        for (auto& e : L->copy_ev) cudaEventDestroy(e);
    }
    host_pipe_destroy(L);
    delete L;
}

int mgpt_moe_num_params(const mgpt_moe_layer* L) { return L ? L->n_params : 0; }

int mgpt_moe_param_shape(const mgpt_moe_layer* L, int i, int* rows, int* cols)
{
    if (!L || !rows || !cols || i < 0 || i >= L->n_params) return fail(MGPT_MOE_EINVAL, "bad parameter index");
    const Dims& d = L->d;
    if (i == 0) { *rows = d.C; *cols = d.E; return 0; }
    if (i == 1) { *rows = 1; *cols = d.E; return 0; }
    switch ((i - 2) % 6) {
        case 0: case 2: *rows = d.C; *cols = d.H; break;
        case 1: case 3: *rows = 1; *cols = d.H; break;
        case 4: *rows = d.H; *cols = d.C; break;
        default: *rows = 1; *cols = d.C; break;
    }
    return 0;
}

int mgpt_moe_bind_params(mgpt_moe_layer* L, float* const* data, float* const* grad, int n)
{
    if (!L || !data) return fail(MGPT_MOE_EINVAL, "null argument");
    // n == 2: router only (the routing side of an expert-parallel layer);
    // n == 2+6E with data[0], data[1] NULL: experts only (the expert side).
    if (n != L->n_params && n != 2) return fail(MGPT_MOE_EINVAL, "expected 2+6E parameter tensors (or the 2 router tensors)");
    const bool router = data[0] != nullptr && data[1] != nullptr;
    const bool experts = n == L->n_params;
    if (!router && !experts) return fail(MGPT_MOE_EINVAL, "null parameter pointer");
    for (int i = 0; i < L->n_params; ++i) {
        const bool want = i < 2 ? router : experts;
        if (want && !data[i]) return fail(MGPT_MOE_EINVAL, "null parameter pointer");
        if (want && grad && !grad[i]) return fail(MGPT_MOE_EINVAL, "null gradient pointer");
        L->p_data[i] = want ? data[i] : nullptr;
        L->p_grad[i] = (want && grad) ? grad[i] : nullptr;
    }
    L->has_grad = grad != nullptr;
    L->router_bound = router;
    L->experts_bound = experts;
    MGPT_CUDA(cudaSetDevice(L->device));
    const int E = L->d.E;
    const size_t CH = (size_t)L->d.C * L->d.H;
    std::vector<void*> h((size_t)15 * E, nullptr);
    for (int e = 0; e < E && experts; ++e) {
        const int b = 2 + 6 * e;
        h[0 * E + e] = data[b + 0]; h[1 * E + e] = data[b + 2]; h[2 * E + e] = data[b + 4];
        h[3 * E + e] = data[b + 1]; h[4 * E + e] = data[b + 3]; h[5 * E + e] = data[b + 5];
        if (grad) {
            h[6 * E + e] = grad[b + 0]; h[7 * E + e] = grad[b + 2]; h[8 * E + e] = grad[b + 4];
            h[9 * E + e] = grad[b + 1]; h[10 * E + e] = grad[b + 3]; h[11 * E + e] = grad[b + 5];
        }
        if (L->sWg) {
            h[12 * E + e] = L->sWg + e * CH; h[13 * E + e] = L->sWu + e * CH; h[14 * E + e] = L->sWd + e * CH;
        }
    }
    MGPT_CUDA(cudaMemcpy(L->d_tables, h.data(), h.size() * sizeof(void*), cudaMemcpyHostToDevice));
    L->bound = router && experts;
    L->shadows_fresh = false;
    L->opt_bound = false;      // the optimiser tables hold the old parameter pointers
    return 0;
}

int mgpt_moe_bind_optimizer_state(mgpt_moe_layer* L, float* const* m, float* const* v, int n)
{
    if (!L || !m || !v) return fail(MGPT_MOE_EINVAL, "null argument");
    if (!L->router_bound && !L->experts_bound) return fail(MGPT_MOE_ESTATE, "bind_params first");
    if (!L->has_grad) return fail(MGPT_MOE_ESTATE, "bind_params with gradient buffers first");
    if (n != L->n_params && n != 2) return fail(MGPT_MOE_EINVAL, "expected 2+6E state tensors (or the 2 router ones)");
    if (L->experts_bound && n != L->n_params) return fail(MGPT_MOE_EINVAL, "expert parameters are bound: pass 2+6E state tensors");
    MGPT_CUDA(cudaSetDevice(L->device));
    const int E = L->d.E, S = E < 2 ? 2 : E;
    if (!L->d_opt) MGPT_CUDA(cudaMalloc(&L->d_opt, (size_t)16 * S * sizeof(void*)));
    std::vector<void*> h((size_t)16 * S, nullptr);
    for (int e = 0; e < E && L->experts_bound; ++e) {
        const int b = 2 + 6 * e;
        const int order[6] = {b + 0, b + 2, b + 4, b + 1, b + 3, b + 5};      // Wg Wu Wd bg bu bd
        for (int j = 0; j < 6; ++j) {
            if (!m[order[j]] || !v[order[j]]) return fail(MGPT_MOE_EINVAL, "null optimiser-state pointer");
            h[(size_t)j * S + e] = m[order[j]];
            h[(size_t)(6 + j) * S + e] = v[order[j]];
        }
    }
    if (L->router_bound) {
        for (int i = 0; i < 2; ++i) {
            if (!m[i] || !v[i]) return fail(MGPT_MOE_EINVAL, "null optimiser-state pointer");
            h[(size_t)12 * S + i] = L->p_data[i];
            h[(size_t)13 * S + i] = L->p_grad[i];
            h[(size_t)14 * S + i] = m[i];
            h[(size_t)15 * S + i] = v[i];
        }
    }
    MGPT_CUDA(cudaMemcpy(L->d_opt, h.data(), h.size() * sizeof(void*), cudaMemcpyHostToDevice));
    L->opt_bound = true;
    return 0;
}

int mgpt_moe_adamw_step(mgpt_moe_layer* L, float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                        mgpt_stream_t stream)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (!L->opt_bound) return fail(MGPT_MOE_ESTATE, "bind_optimizer_state first");
    if (t < 1) return fail(MGPT_MOE_EINVAL, "the step count starts at 1");
    MGPT_CUDA(cudaSetDevice(L->device));
    return launch_adamw(L, lr, beta1, beta2, eps, weight_decay, t, (cudaStream_t)stream);
}

int mgpt_moe_adamw_step_guarded(mgpt_moe_layer* L, float lr, float beta1, float beta2, float eps, float weight_decay,
                                int t, float grad_clip, int skip_nonfinite, mgpt_stream_t stream)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (!L->opt_bound) return fail(MGPT_MOE_ESTATE, "bind_optimizer_state first");
    if (t < 1) return fail(MGPT_MOE_EINVAL, "the step count starts at 1");
    if (!(grad_clip >= 0.0f)) return fail(MGPT_MOE_EINVAL, "grad_clip must be >= 0 (0 = no clamp)");
    MGPT_CUDA(cudaSetDevice(L->device));
    return launch_adamw(L, lr, beta1, beta2, eps, weight_decay, t, (cudaStream_t)stream, grad_clip, skip_nonfinite);
}

int mgpt_moe_sync_weights(mgpt_moe_layer* L, mgpt_stream_t stream)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (!L->router_bound && !L->experts_bound) return fail(MGPT_MOE_ESTATE, "bind_params first");
    MGPT_CUDA(cudaSetDevice(L->device));
    return launch_sync_weights(L, (cudaStream_t)stream);
}

size_t mgpt_moe_workspace_bytes(const mgpt_moe_layer* L, int n_tokens)
{
    if (!L || n_tokens < 0) return 0;
    return make_workspace(L->d, n_tokens).total;
}

int mgpt_moe_workspace_view(const mgpt_moe_layer* L, int n_tokens, const char* name, size_t* offset, size_t* bytes)
{
    if (!L || !name || !offset || !bytes || n_tokens < 0) return fail(MGPT_MOE_EINVAL, "bad argument");
    const Workspace w = make_workspace(L->d, n_tokens);
    const Dims& d = L->d;
    const size_t N = n_tokens, E = d.E, k = d.k, C = d.C, H = d.H, rc = w.row_cap, ab = w.act_bytes;
    struct { const char* n; size_t o, b; } tab[] = {
        {"logits", w.logits, N * E * 4}, {"probs", w.probs, N * E * 4}, {"top_idx", w.top_idx, N * k * 4},
        {"top_p", w.top_p, N * k * 4}, {"counts", w.counts, E * 4}, {"offsets", w.offsets, E * 4},
        {"padded_offsets", w.padded_offsets, (E + 1) * 4}, {"tile_expert", w.tile_expert, (size_t)w.max_tiles * 4},
        {"n_tiles", w.n_tiles, 4}, {"status", w.status, 4}, {"map", w.map, N * k * 4}, {"pos", w.pos, N * k * 4},
        {"row_src", w.row_src, rc * 4}, {"slot", w.slot, N * k * 4}, {"Xg", w.Xg, rc * C * ab}, {"G", w.G, rc * H * ab}, {"U", w.U, rc * H * ab},
        {"Hh", w.Hh, rc * H * ab}, {"Yg", w.Yg, rc * C * ab}, {"dYg", w.dYg, rc * C * ab}, {"dG", w.dG, rc * H * ab},
        {"dU", w.dU, rc * H * ab}, {"dXg", w.dXg, rc * C * ab}, {"d_top_p", w.d_top_p, N * k * 4},
        {"dlogits", w.dlogits, N * E * 4}, {"router_recompute", w.rt_count, 4},
    };
    for (auto& t : tab)
        if (!strcmp(t.n, name)) {
            *offset = t.o;
            *bytes = t.b;
            return 0;
        }
    return fail(MGPT_MOE_EINVAL, std::string("unknown workspace buffer: ") + name);
}

static int check_call(mgpt_moe_layer* L, int n_tokens, int io, const void* ws, size_t ws_bytes, Workspace* w, int kind = 0)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (!L->bound) return fail(MGPT_MOE_ESTATE, "bind_params first (all 2+6E tensors for the whole-layer calls)");
    if (n_tokens < 0) return fail(MGPT_MOE_EINVAL, "negative token count");
    if (io != MGPT_MOE_IO_F32 && io != MGPT_MOE_IO_BF16) return fail(MGPT_MOE_EINVAL, "unknown io dtype");
    if (L->d.mode == MGPT_MOE_FP32 && io != MGPT_MOE_IO_F32) return fail(MGPT_MOE_EINVAL, "FP32 mode takes FP32 tokens");
    if ((long long)n_tokens * L->d.k > (1ll << 30)) return fail(MGPT_MOE_EINVAL, "too many routed rows");
    *w = make_workspace(L->d, n_tokens, kind);
    if (!ws || ((uintptr_t)ws & 255)) return fail(MGPT_MOE_EINVAL, "workspace must be 256-byte aligned");
    if (ws_bytes < w->total) return fail(MGPT_MOE_ENOMEM, "workspace smaller than mgpt_moe_workspace_bytes()");
    if (L->d.mode == MGPT_MOE_BF16 && !L->shadows_fresh)
        return fail(MGPT_MOE_ESTATE, "sync_weights after bind_params / optimiser step");
    return 0;
}

static std::string describe_status(int32_t bits)
{
    std::string m = "a kernel of this layer reported an error since the last check (status " + std::to_string(bits) + "):";
    if (bits & ST_PLAN_OVERFLOW) m += " dispatch plan overflow;";
    if (bits & ST_FULL_WAIT) m += " operand tiles never arrived (bounded wait ran out);";
    if (bits & ST_EMPTY_WAIT) m += " an operand stage was never released (bounded wait ran out);";
    if (bits & ST_ACC_WAIT) m += " an accumulator wait ran out;";
    if (bits & ST_SCHED_WAIT) m += " the work-item queue stalled (bounded wait ran out);";
    if (bits & ST_BAD_EXPERT) m += " an expert id outside [0, num_experts) was skipped;";
    m += " outputs and gradients of the affected step are incomplete";
    return m;
}

// Reads the layer's error word on `st`; the caller synchronises `st` afterwards and calls status_result().
static int status_fetch(mgpt_moe_layer* L, cudaStream_t st)
{
    MGPT_CUDA(cudaMemcpyAsync(L->h_status, L->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    return 0;
}
static int status_result(mgpt_moe_layer* L, cudaStream_t st, int32_t* bits_out)
{
    const int32_t bits = *L->h_status;
    if (bits_out) *bits_out = bits;
    if (bits == 0) return 0;
    cudaMemsetAsync(L->d_status, 0, sizeof(int32_t), st);      // reported once
    return fail(MGPT_MOE_ECUDA, describe_status(bits));
}

int mgpt_moe_check_status(mgpt_moe_layer* L, int32_t* bits)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    MGPT_CUDA(cudaSetDevice(L->device));
    MGPT_TRY(status_fetch(L, L->last_stream));
    MGPT_CUDA(cudaStreamSynchronize(L->last_stream));
    return status_result(L, L->last_stream, bits);
}

int mgpt_moe_selftest_bounded_wait(mgpt_moe_layer* L, mgpt_stream_t stream)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    MGPT_CUDA(cudaSetDevice(L->device));
    return tc_selftest_bounded_wait(L, (cudaStream_t)stream);
}

// Routing results and plan of one forward: the workspace bytes from probs up to (not including) the plan's
// scratch -- probs, top_idx, top_p, counts, offsets, padded_offsets, tile_expert, n_tiles, status, map, pos, row_src,
// pairs, n_pairs.
static size_t routing_begin(const Workspace& w) { return w.probs; }
static size_t routing_end(const Workspace& w) { return w.blk_cnt; }

size_t mgpt_moe_routing_bytes(const mgpt_moe_layer* L, int n_tokens)
{
    if (!L || n_tokens < 0) return 0;
    const Workspace w = make_workspace(L->d, n_tokens);
    return routing_end(w) - routing_begin(w);
}

int mgpt_moe_save_routing(mgpt_moe_layer* L, void* dst, mgpt_stream_t stream)
{
    if (!L || !dst) return fail(MGPT_MOE_EINVAL, "null argument");
    if (!L->fwd_done) return fail(MGPT_MOE_ESTATE, "save_routing without a forward");
    const Workspace w = make_workspace(L->d, L->last_n);
    MGPT_CUDA(cudaSetDevice(L->device));
    MGPT_CUDA(cudaMemcpyAsync(dst, (const char*)L->last_ws + routing_begin(w), routing_end(w) - routing_begin(w),
                              cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return 0;
}

static int forward_impl(mgpt_moe_layer* L, const void* x, void* y, int n_tokens, int io, void* workspace,
                        size_t ws_bytes, mgpt_stream_t stream, const void* routing, const void* residual = nullptr,
                        bool inference = false);

int mgpt_moe_forward(mgpt_moe_layer* L, const void* x, void* y, int n_tokens, int io,
                     void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    return forward_impl(L, x, y, n_tokens, io, workspace, ws_bytes, stream, nullptr);
}

int mgpt_moe_forward_with_routing(mgpt_moe_layer* L, const void* x, void* y, int n_tokens, int io,
                                  void* workspace, size_t ws_bytes, const void* routing, mgpt_stream_t stream)
{
    if (!routing) return fail(MGPT_MOE_EINVAL, "null routing state");
    return forward_impl(L, x, y, n_tokens, io, workspace, ws_bytes, stream, routing);
}

int mgpt_moe_forward_residual(mgpt_moe_layer* L, const void* x, const void* residual, void* y, int n_tokens, int io,
                              void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    if (n_tokens > 0 && !residual) return fail(MGPT_MOE_EINVAL, "null residual");
    return forward_impl(L, x, y, n_tokens, io, workspace, ws_bytes, stream, nullptr, residual);
}

size_t mgpt_moe_inference_workspace_bytes(const mgpt_moe_layer* L, int n_tokens)
{
    if (!L || n_tokens < 0) return 0;
    return make_workspace(L->d, n_tokens, 3).total;
}

int mgpt_moe_forward_inference(mgpt_moe_layer* L, const void* x, void* y, int n_tokens, int io, void* workspace,
                               size_t ws_bytes, mgpt_stream_t stream)
{
    return forward_impl(L, x, y, n_tokens, io, workspace, ws_bytes, stream, nullptr, nullptr, true);
}

static int forward_impl(mgpt_moe_layer* L, const void* x, void* y, int n_tokens, int io, void* workspace,
                        size_t ws_bytes, mgpt_stream_t stream, const void* routing, const void* residual, bool inference)
{
    Workspace w;
    MGPT_TRY(check_call(L, n_tokens, io, workspace, ws_bytes, &w, inference ? 3 : 0));
    if (n_tokens > 0 && (!x || !y)) return fail(MGPT_MOE_EINVAL, "null token buffer");
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const Dims& d = L->d;
    L->fwd_done = false;
    L->ext_Xg = L->ext_Yg = L->ext_dYg = L->ext_dXg = nullptr;      // whole-layer calls keep every buffer in the workspace
    L->n_seg = 0;
    for (int s = 0; s < ST_COUNT; ++s) L->ev_used[s] = false;
    if (routing) {
        // recompute of a forward whose routing was saved: the same tokens route the same way, so router and plan
        // are replaced by one copy (the logits are not part of the saved state and stay undefined)
        L->stage_begin(ST_PLAN, st);
        MGPT_CUDA(cudaMemcpyAsync(ws + routing_begin(w), routing, routing_end(w) - routing_begin(w),
                                  cudaMemcpyDeviceToDevice, st));
        L->stage_end(ST_PLAN, st);
    } else {
        if (n_tokens > 0) {
            L->stage_begin(ST_ROUTER, st);
            if (tc_router_usable(L, x, io, n_tokens))
                MGPT_TRY(tc_router_fwd(L, w, ws, x, st));
            else
                MGPT_TRY(launch_router_fwd(x, io, L->p_data[0], L->p_data[1], n_tokens, d.C, d.E, d.k,
                                           (float*)(ws + w.logits), (float*)(ws + w.probs),
                                           (int32_t*)(ws + w.top_idx), (float*)(ws + w.top_p), st));
            L->stage_end(ST_ROUTER, st);
        }
        L->stage_begin(ST_PLAN, st);
        MGPT_TRY(launch_plan(d, w, ws, st, L->d_status));
        L->stage_end(ST_PLAN, st);
    }
    if (n_tokens > 0) {
        L->stage_begin(ST_DISPATCH, st);
        MGPT_TRY(launch_dispatch(d, w, ws, x, io, st));
        L->stage_end(ST_DISPATCH, st);
        if (use_tc(L)) MGPT_TRY(tc_experts_forward(L, w, ws, st));
        else MGPT_TRY(simt_experts_forward(L, w, ws, st));
        L->stage_begin(ST_COMBINE, st);
        MGPT_TRY(launch_combine_fwd(d, w, ws, y, io, st, residual));
        L->stage_end(ST_COMBINE, st);
    }
    L->last_n = n_tokens;
    L->last_io = io;
    L->last_ws = workspace;
    L->last_stream = st;
    L->fwd_done = !inference;        // nothing was kept: backward cannot follow an inference forward
    L->last_inference = inference;
    return 0;
}

int mgpt_moe_backward(mgpt_moe_layer* L, const void* x, const void* dy, void* dx, int io,
                      void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (!L->fwd_done) return fail(MGPT_MOE_ESTATE, "backward without a forward");
    if (workspace != L->last_ws || io != L->last_io)
        return fail(MGPT_MOE_ESTATE, "backward must reuse the forward's workspace and io dtype");
    Workspace w;
    MGPT_TRY(check_call(L, L->last_n, io, workspace, ws_bytes, &w));
    if (L->last_n == 0) return 0;
    if (!x || !dy || !dx) return fail(MGPT_MOE_EINVAL, "null token buffer");
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    L->stage_begin(ST_COMBINE_BWD, st);
    MGPT_TRY(launch_combine_bwd(L->d, w, ws, dy, io, st));
    L->stage_end(ST_COMBINE_BWD, st);
    // Tensor-core path: the gradients of the rows first, then dx, then the parameter gradients -- dx is what a
    // caller further up the model (or the host, mgpt_moe_step_host) is waiting for, and nothing in the parameter
    // gradients depends on it, so its consumer can start while the largest kernel of the step still runs.
    if (use_tc(L)) MGPT_TRY(tc_experts_backward(L, w, ws, st, 1));
    else MGPT_TRY(simt_experts_backward(L, w, ws, st));
    L->stage_begin(ST_ROUTER_BWD, st);
    MGPT_TRY(launch_router_bwd(L, w, ws, x, io, dx, st));
    L->stage_end(ST_ROUTER_BWD, st);
    if (L->dx_ready_event) MGPT_CUDA(cudaEventRecord(L->dx_ready_event, st));
    if (use_tc(L)) MGPT_TRY(tc_experts_backward(L, w, ws, st, 2));
    if (L->has_grad && !(use_tc(L) && tc_fused_bias_grads(L->d))) {      // else the tensor-core weight-gradient kernel sums the bias gradients itself
        L->stage_begin(ST_BIAS_GRAD, st);
        MGPT_TRY(launch_bias_grads(L, w, ws, st));
        L->stage_end(ST_BIAS_GRAD, st);
    }
    return 0;
}

int mgpt_moe_expert_counts(mgpt_moe_layer* L, int32_t* host_counts)
{
    if (!L || !host_counts) return fail(MGPT_MOE_EINVAL, "null argument");
    if (!L->fwd_done && !L->last_inference) return fail(MGPT_MOE_ESTATE, "no forward has run");
    MGPT_CUDA(cudaSetDevice(L->device));
    const Workspace w = make_workspace(L->d, L->last_n, L->last_inference ? 3 : 0);
    MGPT_CUDA(cudaMemcpyAsync(host_counts, (char*)L->last_ws + w.counts, (size_t)L->d.E * sizeof(int32_t),
                              cudaMemcpyDeviceToHost, L->last_stream));
    MGPT_TRY(status_fetch(L, L->last_stream));
    MGPT_CUDA(cudaStreamSynchronize(L->last_stream));
    return status_result(L, L->last_stream, nullptr);
}

int mgpt_moe_step_host(mgpt_moe_layer* L, const void* x_host, const void* dy_host, void* y_host, void* dx_host,
                       int n_tokens, int io, mgpt_stream_t stream)
{
    if (!L || !x_host || !y_host) return fail(MGPT_MOE_EINVAL, "null argument");
    if (dy_host && !dx_host) return fail(MGPT_MOE_EINVAL, "dx_host is required with dy_host");
    if (n_tokens <= 0) return fail(MGPT_MOE_EINVAL, "n_tokens must be positive");
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    const size_t io_bytes = (size_t)n_tokens * L->d.C * (io == MGPT_MOE_IO_BF16 ? 2 : 4);
    const size_t ws_bytes = mgpt_moe_workspace_bytes(L, n_tokens);
    if (io_bytes > L->h_io_bytes) {             // staging grows on demand, never inside a steady-state step
        MGPT_CUDA(cudaStreamSynchronize(st));
        cudaFree(L->h_x); cudaFree(L->h_dy); cudaFree(L->h_y); cudaFree(L->h_dx);
        L->h_x = L->h_dy = L->h_y = L->h_dx = nullptr;
        L->h_io_bytes = 0;
        MGPT_CUDA(cudaMalloc(&L->h_x, io_bytes));
        MGPT_CUDA(cudaMalloc(&L->h_dy, io_bytes));
        MGPT_CUDA(cudaMalloc(&L->h_y, io_bytes));
        MGPT_CUDA(cudaMalloc(&L->h_dx, io_bytes));
        L->h_io_bytes = io_bytes;
    }
    if (ws_bytes > L->h_ws_bytes) {
        MGPT_CUDA(cudaStreamSynchronize(st));
        cudaFree(L->h_ws);
        L->h_ws = nullptr;
        L->h_ws_bytes = 0;
        MGPT_CUDA(cudaMalloc(&L->h_ws, ws_bytes));
        L->h_ws_bytes = ws_bytes;
    }
    // Copies that nothing is waiting for yet run on a second stream: dy goes up while forward computes and
    // y comes down (the other PCIe direction) while backward computes.
    if (!L->copy_stream) {
        MGPT_CUDA(cudaStreamCreateWithFlags(&L->copy_stream, cudaStreamNonBlocking));
        for (auto& e : L->copy_ev) MGPT_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    cudaStream_t cs = L->copy_stream;
    MGPT_CUDA(cudaMemcpyAsync(L->h_x, x_host, io_bytes, cudaMemcpyHostToDevice, st));
    if (dy_host) {
        MGPT_CUDA(cudaEventRecord(L->copy_ev[0], st));              // after x: keep the upload order x, dy
        MGPT_CUDA(cudaStreamWaitEvent(cs, L->copy_ev[0], 0));
        MGPT_CUDA(cudaMemcpyAsync(L->h_dy, dy_host, io_bytes, cudaMemcpyHostToDevice, cs));
        MGPT_CUDA(cudaEventRecord(L->copy_ev[1], cs));              // dy is on the device
    }
    MGPT_TRY(mgpt_moe_forward(L, L->h_x, L->h_y, n_tokens, io, L->h_ws, L->h_ws_bytes, stream));
    if (dy_host) {
        MGPT_CUDA(cudaEventRecord(L->copy_ev[2], st));              // y is complete
        MGPT_CUDA(cudaStreamWaitEvent(cs, L->copy_ev[2], 0));
        MGPT_CUDA(cudaMemcpyAsync(y_host, L->h_y, io_bytes, cudaMemcpyDeviceToHost, cs));
        MGPT_CUDA(cudaEventRecord(L->copy_ev[3], cs));
        MGPT_CUDA(cudaStreamWaitEvent(st, L->copy_ev[1], 0));       // backward needs dy
        L->dx_ready_event = L->copy_ev[4];                          // recorded inside backward, right after dx is written
        const int brc = mgpt_moe_backward(L, L->h_x, L->h_dy, L->h_dx, io, L->h_ws, L->h_ws_bytes, stream);
        L->dx_ready_event = nullptr;
        MGPT_TRY(brc);
        // dx goes down (after y, same direction) while the parameter gradients are still being formed
        MGPT_CUDA(cudaStreamWaitEvent(cs, L->copy_ev[4], 0));
        MGPT_CUDA(cudaMemcpyAsync(dx_host, L->h_dx, io_bytes, cudaMemcpyDeviceToHost, cs));
        MGPT_CUDA(cudaEventRecord(L->copy_ev[3], cs));
        MGPT_CUDA(cudaStreamWaitEvent(st, L->copy_ev[3], 0));       // the caller's stream also covers both copies
    } else {
        MGPT_CUDA(cudaMemcpyAsync(y_host, L->h_y, io_bytes, cudaMemcpyDeviceToHost, st));
    }
    MGPT_TRY(status_fetch(L, st));
    MGPT_CUDA(cudaStreamSynchronize(st));
    return status_result(L, st, nullptr);
}

// ---- pipelined steps with host buffers ------------------------------------------------------
// One step alone is bound by the PCIe link three times over (x up, y down, dx down; dy goes up beside the forward).
// Consecutive steps do not depend on each other's tokens, so the next step's uploads and the previous step's
// downloads can ride beside this step's kernels: two slots of device staging, one upload stream, one download
// stream, compute on the caller's stream in call order.
}  // extern "C"

namespace {

struct HostSlot {
    void *x = nullptr, *dy = nullptr, *y = nullptr, *dx = nullptr;
    cudaEvent_t in_x = nullptr, in_dy = nullptr, y_ready = nullptr, dx_ready = nullptr, compute_done = nullptr,
                out_done = nullptr;
    bool used = false;                        // a step has been enqueued on this slot and not waited for
};
struct HostPipe {
    HostSlot slot[2];
    size_t io_bytes = 0;
    cudaStream_t up = nullptr, down = nullptr;
    uint64_t n_enqueued = 0;
    cudaStream_t compute = nullptr;           // the stream of the steps in flight
};

void host_pipe_free_slots(HostPipe* hp)
{
    for (auto& s : hp->slot) {
        cudaFree(s.x); cudaFree(s.dy); cudaFree(s.y); cudaFree(s.dx);
        s.x = s.dy = s.y = s.dx = nullptr;
    }
    hp->io_bytes = 0;
}

int host_pipe_drain(mgpt_moe_layer* L, HostPipe* hp)
{
    for (auto& s : hp->slot)
        if (s.used) {
            MGPT_CUDA(cudaEventSynchronize(s.out_done));
            MGPT_CUDA(cudaEventSynchronize(s.compute_done));
            s.used = false;
        }
    (void)L;
    return 0;
}

}  // namespace

void mgpt::host_pipe_destroy(mgpt_moe_layer* L)
{
    HostPipe* hp = (HostPipe*)L->host_pipe;
    if (!hp) return;
    for (auto& s : hp->slot) {
        if (s.used) {
            cudaEventSynchronize(s.out_done);
            cudaEventSynchronize(s.compute_done);
        }
        for (cudaEvent_t e : {s.in_x, s.in_dy, s.y_ready, s.dx_ready, s.compute_done, s.out_done})
            if (e) cudaEventDestroy(e);
    }
    host_pipe_free_slots(hp);
    if (hp->up) cudaStreamDestroy(hp->up);
    if (hp->down) cudaStreamDestroy(hp->down);
    delete hp;
    L->host_pipe = nullptr;
}

extern "C" {

int mgpt_moe_step_host_async(mgpt_moe_layer* L, const void* x_host, const void* dy_host, void* y_host, void* dx_host,
                             int n_tokens, int io, mgpt_stream_t stream)
{
    if (!L || !x_host || !y_host) return fail(MGPT_MOE_EINVAL, "null argument");
    if (dy_host && !dx_host) return fail(MGPT_MOE_EINVAL, "dx_host is required with dy_host");
    if (n_tokens <= 0) return fail(MGPT_MOE_EINVAL, "n_tokens must be positive");
    if (io != MGPT_MOE_IO_F32 && io != MGPT_MOE_IO_BF16) return fail(MGPT_MOE_EINVAL, "unknown io dtype");
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    HostPipe* hp = (HostPipe*)L->host_pipe;
    if (!hp) {
        hp = new HostPipe();
        L->host_pipe = hp;
        int lo = 0, hi = 0;
        MGPT_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        MGPT_CUDA(cudaStreamCreateWithPriority(&hp->up, cudaStreamNonBlocking, hi));
        MGPT_CUDA(cudaStreamCreateWithPriority(&hp->down, cudaStreamNonBlocking, hi));
        for (auto& s : hp->slot)
            for (cudaEvent_t* e : {&s.in_x, &s.in_dy, &s.y_ready, &s.dx_ready, &s.compute_done, &s.out_done})
                MGPT_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
    }
    const size_t io_bytes = (size_t)n_tokens * L->d.C * (io == MGPT_MOE_IO_BF16 ? 2 : 4);
    const size_t ws_bytes = mgpt_moe_workspace_bytes(L, n_tokens);
    if (hp->compute != st || io_bytes > hp->io_bytes || ws_bytes > L->h_ws_bytes) {
        // a new stream or larger buffers: finish what is in flight first (never inside a steady-state loop)
        MGPT_TRY(host_pipe_drain(L, hp));
        hp->compute = st;
    }
    if (io_bytes > hp->io_bytes) {
        host_pipe_free_slots(hp);
        for (auto& s : hp->slot) {
            MGPT_CUDA(cudaMalloc(&s.x, io_bytes));
            MGPT_CUDA(cudaMalloc(&s.dy, io_bytes));
            MGPT_CUDA(cudaMalloc(&s.y, io_bytes));
            MGPT_CUDA(cudaMalloc(&s.dx, io_bytes));
        }
        hp->io_bytes = io_bytes;
    }
    if (ws_bytes > L->h_ws_bytes) {
        MGPT_CUDA(cudaStreamSynchronize(st));
        cudaFree(L->h_ws);
        L->h_ws = nullptr;
        L->h_ws_bytes = 0;
        MGPT_CUDA(cudaMalloc(&L->h_ws, ws_bytes));
        L->h_ws_bytes = ws_bytes;
    }
    HostSlot& s = hp->slot[hp->n_enqueued & 1];
    if (s.used) {
        // the step before last used this slot: its results must be in host memory before its staging is reused
        MGPT_CUDA(cudaEventSynchronize(s.out_done));
        MGPT_CUDA(cudaStreamWaitEvent(hp->up, s.compute_done, 0));       // its backward read x until the end
    }
    ++hp->n_enqueued;
    s.used = true;
    // up: x, then dy, behind the previous step's dy
    MGPT_CUDA(cudaMemcpyAsync(s.x, x_host, io_bytes, cudaMemcpyHostToDevice, hp->up));
    MGPT_CUDA(cudaEventRecord(s.in_x, hp->up));
    if (dy_host) {
        MGPT_CUDA(cudaMemcpyAsync(s.dy, dy_host, io_bytes, cudaMemcpyHostToDevice, hp->up));
        MGPT_CUDA(cudaEventRecord(s.in_dy, hp->up));
    }
    // compute, in call order on the caller's stream
    MGPT_CUDA(cudaStreamWaitEvent(st, s.in_x, 0));
    MGPT_TRY(mgpt_moe_forward(L, s.x, s.y, n_tokens, io, L->h_ws, L->h_ws_bytes, stream));
    MGPT_CUDA(cudaEventRecord(s.y_ready, st));
    // down: y as soon as forward is done, dx as soon as backward has written it (before the weight gradients)
    MGPT_CUDA(cudaStreamWaitEvent(hp->down, s.y_ready, 0));
    MGPT_CUDA(cudaMemcpyAsync(y_host, s.y, io_bytes, cudaMemcpyDeviceToHost, hp->down));
    if (dy_host) {
        MGPT_CUDA(cudaStreamWaitEvent(st, s.in_dy, 0));
        L->dx_ready_event = s.dx_ready;
        const int brc = mgpt_moe_backward(L, s.x, s.dy, s.dx, io, L->h_ws, L->h_ws_bytes, stream);
        L->dx_ready_event = nullptr;
        MGPT_TRY(brc);
        MGPT_CUDA(cudaStreamWaitEvent(hp->down, s.dx_ready, 0));
        MGPT_CUDA(cudaMemcpyAsync(dx_host, s.dx, io_bytes, cudaMemcpyDeviceToHost, hp->down));
    }
    MGPT_CUDA(cudaEventRecord(s.compute_done, st));
    MGPT_CUDA(cudaEventRecord(s.out_done, hp->down));
    return 0;
}

int mgpt_moe_step_host_wait(mgpt_moe_layer* L)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    HostPipe* hp = (HostPipe*)L->host_pipe;
    if (!hp || hp->n_enqueued == 0) return 0;
    MGPT_CUDA(cudaSetDevice(L->device));
    MGPT_TRY(host_pipe_drain(L, hp));
    MGPT_TRY(status_fetch(L, hp->compute));
    MGPT_CUDA(cudaStreamSynchronize(hp->compute));
    return status_result(L, hp->compute, nullptr);
}

static const char* const kStageNames[ST_COUNT] = {
    "router", "plan", "dispatch", "gateup_gemm", "down_gemm", "combine",
    "combine_bwd", "dhh_gemm", "dxg_gemm", "wgrad_gemm", "bias_grad", "router_bwd"};

const char* mgpt_moe_stage_name(int stage)
{
    return (stage >= 0 && stage < ST_COUNT) ? kStageNames[stage] : "";
}

int mgpt_moe_set_weight_grad_overwrite(mgpt_moe_layer* L, int enabled)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (enabled && !use_tc(L)) return fail(MGPT_MOE_EINVAL, "only the tensor-core path (BF16 mode, gemm_impl 0) can overwrite");
    L->bwd_overwrite = enabled != 0;
    return 0;
}

int mgpt_moe_set_sm_budget(mgpt_moe_layer* L, int n_sms)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (n_sms < 0) return fail(MGPT_MOE_EINVAL, "n_sms must be >= 0 (0 = every SM)");
    L->sm_budget = n_sms;
    return 0;
}

int mgpt_moe_set_profiling(mgpt_moe_layer* L, int enabled)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    MGPT_CUDA(cudaSetDevice(L->device));
    if (enabled && !L->ev_begin[0]) {
        for (int s = 0; s < ST_COUNT; ++s) {
            MGPT_CUDA(cudaEventCreate(&L->ev_begin[s]));
            MGPT_CUDA(cudaEventCreate(&L->ev_end[s]));
        }
    }
    L->profiling = enabled != 0;
    return 0;
}

int mgpt_moe_stage_ms(mgpt_moe_layer* L, float* ms)
{
    if (!L || !ms) return fail(MGPT_MOE_EINVAL, "null argument");
    for (int s = 0; s < ST_COUNT; ++s) {
        ms[s] = 0.0f;
        if (!L->ev_used[s]) continue;
        MGPT_CUDA(cudaEventSynchronize(L->ev_end[s]));
        MGPT_CUDA(cudaEventElapsedTime(&ms[s], L->ev_begin[s], L->ev_end[s]));
    }
    // the stages just waited for have finished: a time measured on a step that reported an error is not a time
    MGPT_CUDA(cudaMemcpy(L->h_status, L->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost));
    return status_result(L, L->last_stream, nullptr);
}

int mgpt_moe_op_router(const void* x, int io, const float* Wr, const float* br, int n_tokens, int C, int E, int k,
                       float* logits, float* probs, int32_t* top_idx, float* top_p, mgpt_stream_t stream)
{
    if (!x || !Wr || !br || !probs || !top_idx || !top_p) return fail(MGPT_MOE_EINVAL, "null argument");
    if (E <= 0 || E > MAX_EXPERTS || k <= 0 || k > MAX_TOPK || k > E || C <= 0 || n_tokens < 0)
        return fail(MGPT_MOE_EINVAL, "unsupported router shape");
    return launch_router_fwd(x, io, Wr, br, n_tokens, C, E, k, logits, probs, top_idx, top_p, (cudaStream_t)stream);
}

}  // extern "C"
