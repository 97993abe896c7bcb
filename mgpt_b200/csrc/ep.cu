// Expert parallelism behind the C ABI: one routing-side layer, one expert-side layer per chunk of local experts,
// and the exchange of rows between ranks over NCCL point-to-point calls on a stream of its own.
//
// The reference has no multi-GPU code; what is sharded here is the expert loop of MoELayer::forward_into /
// backward_into (layers/MoELayer.cpp:94-118, 159-181).  The stage-level entry points of stages.cu do all the
// arithmetic; this file only moves rows and keeps the two streams in step:
//
//   forward   route | counts <-> | rows -> (all chunks queued at once) | per chunk: experts, rows <- | combine
//   backward  combine_backward | rows -> | per chunk: experts' row gradients, rows <-, parameter gradients | route_backward
//
// Rows travel in the padded expert-major layout (every expert's segment a whole number of 128-row tiles), so the
// block for a peer is one contiguous range and what arrives is computed on where it lands.
// NCCL is loaded with dlopen("libnccl.so.2") at the first use: a process that already has it (torch) shares that
// copy, a single-GPU process never needs it.
#include <dlfcn.h>

#include <cstring>
#include <vector>

#include "common.cuh"

using namespace mgpt;

namespace {

// ---- the few NCCL entry points used, resolved at run time ---------------------------------------------------------
typedef struct { char internal[128]; } NcclUniqueId;
typedef void* NcclComm;
struct Nccl {
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*Send)(const void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};
Nccl g_nccl;

int load_nccl()
{
    if (g_nccl.ok) return 0;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(MGPT_MOE_ECUDA, std::string("expert parallelism over more than one rank needs NCCL: ") + dlerror());
#define MGPT_SYM(field, name)                                                                  \
    *(void**)(&g_nccl.field) = dlsym(h, name);                                                 \
    if (!g_nccl.field) return fail(MGPT_MOE_ECUDA, std::string("libnccl has no symbol ") + name)
    MGPT_SYM(GetUniqueId, "ncclGetUniqueId");
    MGPT_SYM(CommInitRank, "ncclCommInitRank");
    MGPT_SYM(CommDestroy, "ncclCommDestroy");
    MGPT_SYM(Send, "ncclSend");
    MGPT_SYM(Recv, "ncclRecv");
    MGPT_SYM(GroupStart, "ncclGroupStart");
    MGPT_SYM(GroupEnd, "ncclGroupEnd");
    MGPT_SYM(AllGather, "ncclAllGather");
    MGPT_SYM(AllReduce, "ncclAllReduce");
    MGPT_SYM(GetErrorString, "ncclGetErrorString");
#undef MGPT_SYM
    g_nccl.ok = true;
    return 0;
}

int nccl_fail(int rc, const char* what)
{
    return fail(MGPT_MOE_ECUDA, std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "NCCL error"));
}
#define MGPT_NCCL(call)                                    \
    do {                                                   \
        int rc__ = (call);                                 \
        if (rc__ != 0) return nccl_fail(rc__, #call);      \
    } while (0)

constexpr int NCCL_BYTES = 0;      // ncclInt8: every message is sent as bytes
constexpr int NCCL_INT32 = 2, NCCL_SUM = 0;
constexpr int IPC_BYTES = 64;      // cudaIpcMemHandle_t

inline int pad128(int v) { return (v + ROW_TILE - 1) / ROW_TILE * ROW_TILE; }

struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    int ensure(size_t need)
    {
        if (need <= bytes) return 0;
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
        MGPT_CUDA(cudaMalloc(&p, need ? need : 256));
        bytes = need ? need : 256;
        return 0;
    }
    void release()
    {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
};

}  // namespace

struct mgpt_moe_ep {
    mgpt_moe_ep_config cfg;
    int C, H, E, k, G, rank, nc, E_local, E_chunk;
    size_t act;                                   // bytes per row element (2 in BF16 mode, 4 in FP32 mode)
    mgpt_moe_layer* home = nullptr;
    std::vector<mgpt_moe_layer*> locals;
    NcclComm comm = nullptr;
    cudaStream_t cs = nullptr;                    // exchange stream
    cudaEvent_t ev_main = nullptr;                // "the compute stream has reached this point"
    std::vector<cudaEvent_t> ev_in, ev_out, ev_back;
    // device buffers
    DevBuf home_ws, rows, rows_back, d_rows, d_back, recv_counts;
    std::vector<DevBuf> recv_rows, out_rows, d_recv, d_in, local_ws, seg_counts;
    // host copies of the counts (pinned) and the split sizes of the last forward
    int32_t *h_counts = nullptr, *h_recv = nullptr;
    std::vector<std::vector<int>> send_split, recv_split;     // [chunk][peer] padded rows
    std::vector<int> starts, n_recv;                          // first send row / received rows of a chunk
    int n_send = 0, last_n = 0, last_io = 0;
    bool fwd_done = false;
    // copy-engine transport (cfg.max_tokens > 0): four buffers of this rank that the peers read (rows routed here,
    // expert outputs, and their gradient mirrors), the peers' mappings of theirs, local landing buffers
    bool peer = false;
    size_t cap_send = 0, cap_recv = 0;            // rows
    void* pb[4] = {nullptr, nullptr, nullptr, nullptr};       // A rows, B outputs, Cg row gradients, D input gradients
    std::vector<void*> peer_ptr[4];               // [rank] -> that rank's buffer as mapped here (own: pb[i])
    DevBuf recv_all, drecv_all, every, flag;
    int32_t* h_every = nullptr;                   // pinned [G][E]: every rank's counts
    std::vector<int> blk, send_off, recv_off;     // [s][d][c] rows; [s][c][d] first row in s's send layout; [d][c][s] in d's receive layout
    std::vector<int> recv_base;                   // [c] first row of chunk c in this rank's receive layout
};

namespace {

// recv[g] <- send[g] for every peer g: row ranges given as {first row, rows} per peer; enqueued on the exchange stream
int exchange_rows(mgpt_moe_ep* ep, char* recv, const std::vector<int>& recv_n, const char* send,
                  const std::vector<int>& send_n)
{
    const size_t rb = (size_t)ep->C * ep->act;
    size_t so = 0, ro = 0;
    if (ep->G > 1) MGPT_NCCL(g_nccl.GroupStart());
    for (int g = 0; g < ep->G; ++g) {
        const size_t sbytes = (size_t)send_n[g] * rb, rbytes = (size_t)recv_n[g] * rb;
        if (g == ep->rank) {
            if (sbytes) MGPT_CUDA(cudaMemcpyAsync(recv + ro, send + so, sbytes, cudaMemcpyDeviceToDevice, ep->cs));
        } else {
            if (sbytes) MGPT_NCCL(g_nccl.Send(send + so, sbytes, NCCL_BYTES, g, ep->comm, ep->cs));
            if (rbytes) MGPT_NCCL(g_nccl.Recv(recv + ro, rbytes, NCCL_BYTES, g, ep->comm, ep->cs));
        }
        so += sbytes;
        ro += rbytes;
    }
    if (ep->G > 1) MGPT_NCCL(g_nccl.GroupEnd());
    return 0;
}

// the exchange stream continues only after everything enqueued on `st` so far
int follow(mgpt_moe_ep* ep, cudaStream_t st)
{
    MGPT_CUDA(cudaEventRecord(ep->ev_main, st));
    MGPT_CUDA(cudaStreamWaitEvent(ep->cs, ep->ev_main, 0));
    return 0;
}

// every rank's kernels enqueued on `st` so far are complete on every rank before what is enqueued on `st` afterwards
int barrier_on(mgpt_moe_ep* ep, cudaStream_t st)
{
    MGPT_NCCL(g_nccl.AllReduce(ep->flag.p, ep->flag.p, 1, NCCL_INT32, NCCL_SUM, ep->comm, st));
    return 0;
}

// this rank's blocks of chunk c, pulled from the producers' buffers `which` into `dst` (receive layout) -- or, with
// back = true, this rank's rows of chunk c pulled back from the owners' buffers into `dst` (send layout)
int pull_chunk(mgpt_moe_ep* ep, int which, char* dst, int c, bool back)
{
    const int G = ep->G, nc = ep->nc, me = ep->rank;
    const size_t rb = (size_t)ep->C * ep->act;
    for (int i = 0; i < G; ++i) {
        const int o = (me + i) % G;                  // every rank starts at a different peer
        size_t d_row, s_row, rows;
        if (!back) {
            rows = ep->blk[((size_t)o * G + me) * nc + c];
            d_row = ep->recv_off[((size_t)me * nc + c) * G + o];
            s_row = ep->send_off[((size_t)o * nc + c) * G + me];
        } else {
            rows = ep->blk[((size_t)me * G + o) * nc + c];
            d_row = ep->send_off[((size_t)me * nc + c) * G + o];
            s_row = ep->recv_off[((size_t)o * nc + c) * G + me];
        }
        if (rows)
            MGPT_CUDA(cudaMemcpyAsync(dst + d_row * rb, (const char*)ep->peer_ptr[which][o] + s_row * rb, rows * rb,
                                      cudaMemcpyDeviceToDevice, ep->cs));
    }
    return 0;
}

int sum(const std::vector<int>& v)
{
    int s = 0;
    for (int x : v) s += x;
    return s;
}

}  // namespace

namespace {

// Allocates the peer-readable buffers, all-gathers their IPC handles over NCCL and maps the peers' buffers.
int setup_peer(mgpt_moe_ep* ep)
{
    const int G = ep->G;
    const size_t rb = (size_t)ep->C * ep->act;
    size_t off = 0, nb = 0;
    MGPT_TRY(mgpt_moe_workspace_view(ep->home, ep->cfg.max_tokens, "row_src", &off, &nb));
    ep->cap_send = nb / sizeof(int32_t);
    ep->cap_recv = (size_t)G * ep->cap_send;       // worst case: every rank routes all of its rows here
    const size_t bytes[4] = {ep->cap_send * rb, ep->cap_recv * rb, ep->cap_send * rb, ep->cap_recv * rb};
    std::vector<char> mine(4 * IPC_BYTES), all((size_t)G * 4 * IPC_BYTES);
    for (int i = 0; i < 4; ++i) {
        MGPT_CUDA(cudaMalloc(&ep->pb[i], bytes[i]));
        cudaIpcMemHandle_t h;
        MGPT_CUDA(cudaIpcGetMemHandle(&h, ep->pb[i]));
        static_assert(sizeof(h) == IPC_BYTES, "handle size");
        memcpy(mine.data() + i * IPC_BYTES, &h, IPC_BYTES);
    }
    DevBuf d_mine, d_all;
    MGPT_TRY(d_mine.ensure(mine.size()));
    MGPT_TRY(d_all.ensure(all.size()));
    MGPT_CUDA(cudaMemcpyAsync(d_mine.p, mine.data(), mine.size(), cudaMemcpyHostToDevice, ep->cs));
    int nrc = g_nccl.AllGather(d_mine.p, d_all.p, mine.size(), NCCL_BYTES, ep->comm, ep->cs);
    if (nrc == 0) {
        cudaMemcpyAsync(all.data(), d_all.p, all.size(), cudaMemcpyDeviceToHost, ep->cs);
        cudaStreamSynchronize(ep->cs);
    }
    d_mine.release();
    d_all.release();
    if (nrc != 0) return nccl_fail(nrc, "ncclAllGather(handles)");
    for (int i = 0; i < 4; ++i) {
        ep->peer_ptr[i].assign(G, nullptr);
        for (int g = 0; g < G; ++g) {
            if (g == ep->rank) {
                ep->peer_ptr[i][g] = ep->pb[i];
                continue;
            }
            cudaIpcMemHandle_t h;
            memcpy(&h, all.data() + ((size_t)g * 4 + i) * IPC_BYTES, IPC_BYTES);
            MGPT_CUDA(cudaIpcOpenMemHandle(&ep->peer_ptr[i][g], h, cudaIpcMemLazyEnablePeerAccess));
        }
    }
    MGPT_TRY(ep->recv_all.ensure(ep->cap_recv * rb));
    MGPT_TRY(ep->drecv_all.ensure(ep->cap_recv * rb));
    MGPT_TRY(ep->rows_back.ensure(ep->cap_send * rb));
    MGPT_TRY(ep->d_back.ensure(ep->cap_send * rb));
    MGPT_TRY(ep->every.ensure((size_t)G * ep->E * sizeof(int32_t)));
    MGPT_TRY(ep->flag.ensure(256));
    MGPT_CUDA(cudaMemsetAsync(ep->flag.p, 0, 256, ep->cs));
    MGPT_CUDA(cudaHostAlloc(&ep->h_every, (size_t)G * ep->E * sizeof(int32_t), cudaHostAllocDefault));
    MGPT_CUDA(cudaStreamSynchronize(ep->cs));
    ep->blk.assign((size_t)G * G * ep->nc, 0);
    ep->send_off.assign((size_t)G * ep->nc * G, 0);
    ep->recv_off.assign((size_t)G * ep->nc * G, 0);
    ep->recv_base.assign(ep->nc, 0);
    ep->peer = true;
    return 0;
}

// forward with the copy-engine transport (see mgpt_moe_ep_config::max_tokens)
int forward_peer(mgpt_moe_ep* ep, const void* x, void* y, int n_tokens, int io, mgpt_stream_t stream)
{
    cudaStream_t st = (cudaStream_t)stream;
    const int G = ep->G, nc = ep->nc, Ec = ep->E_chunk, E = ep->E, me = ep->rank;
    const size_t rb = (size_t)ep->C * ep->act;
    if (n_tokens > ep->cfg.max_tokens) return fail(MGPT_MOE_EINVAL, "n_tokens exceeds the max_tokens the layer was created with");
    const size_t home_bytes = mgpt_moe_stage_workspace_bytes(ep->home, n_tokens, 1);
    MGPT_TRY(ep->home_ws.ensure(home_bytes));
    MGPT_TRY(mgpt_moe_route_plan(ep->home, x, n_tokens, io, ep->home_ws.p, ep->home_ws.bytes, stream));
    size_t off = 0, nb = 0;
    MGPT_TRY(mgpt_moe_workspace_view(ep->home, n_tokens, "counts", &off, &nb));
    const int32_t* d_counts = (const int32_t*)((char*)ep->home_ws.p + off);
    // every rank's counts to every rank (global expert order = chunk, owner, j), while the rows are permuted
    MGPT_TRY(follow(ep, st));
    MGPT_TRY(mgpt_moe_route_rows(ep->home, x, io, ep->home_ws.p, ep->home_ws.bytes, ep->pb[0], stream));
    MGPT_NCCL(g_nccl.AllGather(d_counts, ep->every.p, (size_t)E * sizeof(int32_t), NCCL_BYTES, ep->comm, ep->cs));
    MGPT_CUDA(cudaMemcpyAsync(ep->h_every, ep->every.p, (size_t)G * E * sizeof(int32_t), cudaMemcpyDeviceToHost, ep->cs));
    MGPT_CUDA(cudaStreamSynchronize(ep->cs));               // the one host synchronisation: how many rows go where
    auto M = [&](int s, int c, int d, int j) { return ep->h_every[(size_t)s * E + (c * G + d) * Ec + j]; };
    for (int s = 0; s < G; ++s)
        for (int d = 0; d < G; ++d)
            for (int c = 0; c < nc; ++c) {
                int rows = 0;
                for (int j = 0; j < Ec; ++j) rows += pad128(M(s, c, d, j));
                ep->blk[((size_t)s * G + d) * nc + c] = rows;
            }
    for (int r = 0; r < G; ++r) {
        int so = 0, ro = 0;
        for (int c = 0; c < nc; ++c)
            for (int o = 0; o < G; ++o) {
                ep->send_off[((size_t)r * nc + c) * G + o] = so;
                so += ep->blk[((size_t)r * G + o) * nc + c];
                ep->recv_off[((size_t)r * nc + c) * G + o] = ro;
                ro += ep->blk[((size_t)o * G + r) * nc + c];
            }
    }
    ep->n_send = 0;
    for (int c = 0; c < nc; ++c) {
        ep->starts[c] = ep->send_off[((size_t)me * nc + c) * G];
        ep->recv_base[c] = ep->recv_off[((size_t)me * nc + c) * G];
        ep->n_recv[c] = 0;
        for (int o = 0; o < G; ++o) {
            ep->n_recv[c] += ep->blk[((size_t)o * G + me) * nc + c];
            ep->n_send += ep->blk[((size_t)me * G + o) * nc + c];
            for (int j = 0; j < Ec; ++j) ep->h_recv[(o * nc + c) * Ec + j] = M(o, c, me, j);
        }
    }
    for (int c = 0; c < nc; ++c) {
        MGPT_TRY(ep->local_ws[c].ensure(mgpt_moe_stage_workspace_bytes(ep->locals[c], ep->n_recv[c], 0)));
        MGPT_TRY(ep->seg_counts[c].ensure((size_t)G * Ec * sizeof(int32_t)));
        // real counts per (source, local expert of chunk c): column block (c, me) of every source's row of counts
        MGPT_CUDA(cudaMemcpy2DAsync(ep->seg_counts[c].p, Ec * sizeof(int32_t), (const int32_t*)ep->every.p + (c * G + me) * Ec,
                                    (size_t)E * sizeof(int32_t), Ec * sizeof(int32_t), G, cudaMemcpyDeviceToDevice, ep->cs));
    }
    // the permuted rows of every rank are complete: route_rows was enqueued after the all-gather's snapshot of the
    // compute stream, so it gets a barrier of its own (the compute stream is idle here, the barrier starts at once)
    MGPT_TRY(follow(ep, st));
    MGPT_TRY(barrier_on(ep, ep->cs));
    for (int c = 0; c < nc; ++c) {
        MGPT_TRY(pull_chunk(ep, 0, (char*)ep->recv_all.p, c, false));
        MGPT_CUDA(cudaEventRecord(ep->ev_in[c], ep->cs));
    }
    for (int c = 0; c < nc; ++c) {
        char* in = (char*)ep->recv_all.p + (size_t)ep->recv_base[c] * rb;
        char* out = (char*)ep->pb[1] + (size_t)ep->recv_base[c] * rb;
        MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_in[c], 0));
        MGPT_TRY(mgpt_moe_experts_forward(ep->locals[c], in, (const int32_t*)ep->seg_counts[c].p, G, ep->n_recv[c], out,
                                          ep->local_ws[c].p, ep->local_ws[c].bytes, stream));
        // barrier in the order of the compute stream (beside it, its kernel would wait for the next persistent
        // kernel to end), then the copies it releases run beside the next chunk's products
        MGPT_TRY(barrier_on(ep, st));
        MGPT_CUDA(cudaEventRecord(ep->ev_out[c], st));
        MGPT_CUDA(cudaStreamWaitEvent(ep->cs, ep->ev_out[c], 0));
        MGPT_TRY(pull_chunk(ep, 1, (char*)ep->rows_back.p, c, true));
        MGPT_CUDA(cudaEventRecord(ep->ev_back[c], ep->cs));
    }
    MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_back[nc - 1], 0));
    MGPT_TRY(mgpt_moe_combine(ep->home, ep->rows_back.p, y, io, ep->home_ws.p, ep->home_ws.bytes, stream));
    ep->last_n = n_tokens;
    ep->last_io = io;
    ep->fwd_done = true;
    return 0;
}

int backward_peer(mgpt_moe_ep* ep, const void* x, const void* dy, void* dx, int io, mgpt_stream_t stream)
{
    cudaStream_t st = (cudaStream_t)stream;
    const int nc = ep->nc;
    const size_t rb = (size_t)ep->C * ep->act;
    MGPT_TRY(mgpt_moe_combine_backward(ep->home, ep->rows_back.p, dy, io, ep->pb[2], ep->home_ws.p, ep->home_ws.bytes, stream));
    MGPT_TRY(barrier_on(ep, st));                    // every rank's row gradients are written
    MGPT_TRY(follow(ep, st));
    for (int c = 0; c < nc; ++c) {
        MGPT_TRY(pull_chunk(ep, 2, (char*)ep->drecv_all.p, c, false));
        MGPT_CUDA(cudaEventRecord(ep->ev_in[c], ep->cs));
    }
    for (int c = 0; c < nc; ++c) {
        char* d_out = (char*)ep->drecv_all.p + (size_t)ep->recv_base[c] * rb;
        char* d_in = (char*)ep->pb[3] + (size_t)ep->recv_base[c] * rb;
        MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_in[c], 0));
        MGPT_TRY(mgpt_moe_experts_backward_rows(ep->locals[c], d_out, d_in, ep->local_ws[c].p, ep->local_ws[c].bytes, stream));
        MGPT_TRY(barrier_on(ep, st));
        MGPT_CUDA(cudaEventRecord(ep->ev_out[c], st));
        MGPT_CUDA(cudaStreamWaitEvent(ep->cs, ep->ev_out[c], 0));
        MGPT_TRY(pull_chunk(ep, 3, (char*)ep->d_back.p, c, true));
        MGPT_CUDA(cudaEventRecord(ep->ev_back[c], ep->cs));
        MGPT_TRY(mgpt_moe_experts_backward_params(ep->locals[c], d_out, d_in, ep->local_ws[c].p, ep->local_ws[c].bytes, stream));
    }
    MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_back[nc - 1], 0));
    return mgpt_moe_route_backward(ep->home, x, ep->d_back.p, dx, io, ep->home_ws.p, ep->home_ws.bytes, stream);
}

}  // namespace

extern "C" {

int mgpt_moe_ep_unique_id(void* id_out)
{
    if (!id_out) return fail(MGPT_MOE_EINVAL, "null argument");
    MGPT_TRY(load_nccl());
    NcclUniqueId id;
    MGPT_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id_out, &id, sizeof(id));
    return 0;
}

void mgpt_moe_ep_destroy(mgpt_moe_ep* ep)
{
    if (!ep) return;
    cudaSetDevice(ep->cfg.device);
    cudaDeviceSynchronize();
    if (ep->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ep->comm);
    mgpt_moe_destroy(ep->home);
    for (auto* l : ep->locals) mgpt_moe_destroy(l);
    for (DevBuf* b : {&ep->home_ws, &ep->rows, &ep->rows_back, &ep->d_rows, &ep->d_back, &ep->recv_counts}) b->release();
    for (auto* v : {&ep->recv_rows, &ep->out_rows, &ep->d_recv, &ep->d_in, &ep->local_ws, &ep->seg_counts})
        for (auto& b : *v) b.release();
    for (int i = 0; i < 4; ++i) {
        for (int g = 0; g < (int)ep->peer_ptr[i].size(); ++g)
            if (g != ep->rank && ep->peer_ptr[i][g]) cudaIpcCloseMemHandle(ep->peer_ptr[i][g]);
    }
    if (ep->peer && ep->comm && g_nccl.AllReduce && ep->flag.p) {
        // every rank has closed its mappings before any rank frees what they pointed at
        g_nccl.AllReduce(ep->flag.p, ep->flag.p, 1, NCCL_INT32, NCCL_SUM, ep->comm, ep->cs);
        cudaStreamSynchronize(ep->cs);
    }
    for (int i = 0; i < 4; ++i)
        if (ep->pb[i]) cudaFree(ep->pb[i]);
    for (DevBuf* b : {&ep->recv_all, &ep->drecv_all, &ep->every, &ep->flag}) b->release();
    if (ep->h_every) cudaFreeHost(ep->h_every);
    if (ep->h_counts) cudaFreeHost(ep->h_counts);
    if (ep->h_recv) cudaFreeHost(ep->h_recv);
    for (auto* v : {&ep->ev_in, &ep->ev_out, &ep->ev_back})
        for (auto e : *v) cudaEventDestroy(e);
    if (ep->ev_main) cudaEventDestroy(ep->ev_main);
    if (ep->cs) cudaStreamDestroy(ep->cs);
    delete ep;
}

int mgpt_moe_ep_create(const mgpt_moe_ep_config* cfg, const void* id, mgpt_moe_ep** out)
{
    if (!cfg || !out) return fail(MGPT_MOE_EINVAL, "null argument");
    const int G = cfg->world, nc = cfg->n_chunks < 1 ? 1 : cfg->n_chunks;
    if (G < 1 || cfg->rank < 0 || cfg->rank >= G) return fail(MGPT_MOE_EINVAL, "rank must be in [0, world)");
    if (cfg->num_experts % G) return fail(MGPT_MOE_EINVAL, "num_experts is not divisible by the number of ranks");
    if ((cfg->num_experts / G) % nc) return fail(MGPT_MOE_EINVAL, "the experts of a rank do not split into n_chunks chunks");
    if (G > MAX_SOURCES) return fail(MGPT_MOE_EINVAL, "at most 64 ranks");
    if (G > 1 && !id) return fail(MGPT_MOE_EINVAL, "null NCCL id");
    mgpt_moe_ep* ep = new mgpt_moe_ep();
    ep->cfg = *cfg;
    ep->cfg.n_chunks = nc;
    ep->C = cfg->embed_dim;
    ep->H = cfg->hidden_dim == -1 ? 4 * cfg->embed_dim : cfg->hidden_dim;
    ep->E = cfg->num_experts; ep->k = cfg->top_k; ep->G = G; ep->rank = cfg->rank; ep->nc = nc;
    ep->E_local = ep->E / G;
    ep->E_chunk = ep->E_local / nc;
    ep->act = cfg->mode == MGPT_MOE_BF16 ? 2 : 4;
    auto bail = [&](int rc) {
        mgpt_moe_ep_destroy(ep);
        return rc;
    };
    mgpt_moe_config hc = {cfg->embed_dim, cfg->hidden_dim, cfg->num_experts, cfg->top_k, cfg->lb_alpha, cfg->mode, cfg->device, 0};
    int rc = mgpt_moe_create(&hc, &ep->home);
    if (rc) return bail(rc);
    for (int c = 0; c < nc; ++c) {
        mgpt_moe_config lc = {cfg->embed_dim, cfg->hidden_dim, ep->E_chunk, 1, cfg->lb_alpha, cfg->mode, cfg->device, 0};
        mgpt_moe_layer* l = nullptr;
        rc = mgpt_moe_create(&lc, &l);
        if (rc) return bail(rc);
        ep->locals.push_back(l);
    }
    // The exchange stream gets the highest priority: when an exchange and a persistent compute kernel become ready at
    // the same moment, the exchange's few CTAs are placed first and the compute CTAs that find their SM taken start
    // late and simply take fewer work items; the other way round the exchange would wait for the whole kernel.
    int prio_lo = 0, prio_hi = 0;
    cudaError_t e = cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&ep->cs, cudaStreamNonBlocking, prio_hi);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ep->ev_main, cudaEventDisableTiming);
    for (auto* v : {&ep->ev_in, &ep->ev_out, &ep->ev_back})
        for (int c = 0; c < nc && e == cudaSuccess; ++c) {
            cudaEvent_t ev;
            e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
            if (e == cudaSuccess) v->push_back(ev);
        }
    if (e == cudaSuccess) e = cudaHostAlloc(&ep->h_counts, (size_t)ep->E * sizeof(int32_t), cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaHostAlloc(&ep->h_recv, (size_t)ep->E * sizeof(int32_t), cudaHostAllocDefault);
    if (e != cudaSuccess) return bail(cuda_fail(e, "expert-parallel layer set-up"));
    ep->recv_rows.resize(nc); ep->out_rows.resize(nc); ep->d_recv.resize(nc); ep->d_in.resize(nc);
    ep->local_ws.resize(nc); ep->seg_counts.resize(nc);
    ep->send_split.assign(nc, std::vector<int>(G, 0));
    ep->recv_split.assign(nc, std::vector<int>(G, 0));
    ep->starts.assign(nc, 0);
    ep->n_recv.assign(nc, 0);
    if (G > 1) {
        rc = load_nccl();
        if (rc) return bail(rc);
        NcclUniqueId uid;
        memcpy(&uid, id, sizeof(uid));
        int nrc = g_nccl.CommInitRank(&ep->comm, G, uid, cfg->rank);
        if (nrc != 0) return bail(nccl_fail(nrc, "ncclCommInitRank"));
    }
    if (G > 1 && cfg->max_tokens > 0) {
        rc = setup_peer(ep);
        if (rc) return bail(rc);
    }
    *out = ep;
    return 0;
}

int mgpt_moe_ep_num_params(const mgpt_moe_ep* ep) { return ep ? 2 + 6 * ep->E_local : 0; }

int mgpt_moe_ep_global_expert(const mgpt_moe_ep* ep, int l)
{
    if (!ep || l < 0 || l >= ep->E_local) return -1;
    const int c = l / ep->E_chunk, j = l % ep->E_chunk;
    return c * (ep->E / ep->nc) + ep->rank * ep->E_chunk + j;
}

int mgpt_moe_ep_bind_params(mgpt_moe_ep* ep, float* const* data, float* const* grad, int n)
{
    if (!ep || !data) return fail(MGPT_MOE_EINVAL, "null argument");
    if (n != 2 + 6 * ep->E_local) return fail(MGPT_MOE_EINVAL, "expected 2 + 6*E/world parameter tensors");
    MGPT_TRY(mgpt_moe_bind_params(ep->home, data, grad, 2));
    const int per = 6 * ep->E_chunk;
    for (int c = 0; c < ep->nc; ++c) {
        std::vector<float*> d(2 + per, nullptr), g(2 + per, nullptr);
        for (int i = 0; i < per; ++i) {
            d[2 + i] = data[2 + c * per + i];
            if (grad) g[2 + i] = grad[2 + c * per + i];
        }
        MGPT_TRY(mgpt_moe_bind_params(ep->locals[c], d.data(), grad ? g.data() : nullptr, 2 + per));
    }
    return 0;
}

int mgpt_moe_ep_sync_weights(mgpt_moe_ep* ep, mgpt_stream_t stream)
{
    if (!ep) return fail(MGPT_MOE_EINVAL, "null argument");
    MGPT_TRY(mgpt_moe_sync_weights(ep->home, stream));
    for (auto* l : ep->locals) MGPT_TRY(mgpt_moe_sync_weights(l, stream));
    return 0;
}

int mgpt_moe_ep_check_status(mgpt_moe_ep* ep)
{
    if (!ep) return fail(MGPT_MOE_EINVAL, "null argument");
    MGPT_TRY(mgpt_moe_check_status(ep->home, nullptr));
    for (auto* l : ep->locals) MGPT_TRY(mgpt_moe_check_status(l, nullptr));
    return 0;
}

int mgpt_moe_ep_received_counts(mgpt_moe_ep* ep, int32_t* out)
{
    if (!ep || !out) return fail(MGPT_MOE_EINVAL, "null argument");
    if (!ep->fwd_done) return fail(MGPT_MOE_ESTATE, "no forward has run");
    for (int g = 0; g < ep->G; ++g)
        for (int c = 0; c < ep->nc; ++c)
            for (int j = 0; j < ep->E_chunk; ++j)
                out[g * ep->E_local + c * ep->E_chunk + j] = ep->h_recv[(g * ep->nc + c) * ep->E_chunk + j];
    return 0;
}

}  // extern "C"

extern "C" {

int mgpt_moe_ep_forward(mgpt_moe_ep* ep, const void* x, void* y, int n_tokens, int io, mgpt_stream_t stream)
{
    if (!ep) return fail(MGPT_MOE_EINVAL, "null argument");
    if (n_tokens <= 0 || !x || !y) return fail(MGPT_MOE_EINVAL, "bad token buffer");
    MGPT_CUDA(cudaSetDevice(ep->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const int G = ep->G, nc = ep->nc, Ec = ep->E_chunk;
    const size_t rb = (size_t)ep->C * ep->act;
    ep->fwd_done = false;
    if (ep->peer) return forward_peer(ep, x, y, n_tokens, io, stream);

    // routing side: router, plan, rows in the padded expert-major layout (experts in global order = chunk, rank, j)
    const size_t home_bytes = mgpt_moe_stage_workspace_bytes(ep->home, n_tokens, 1);
    MGPT_TRY(ep->home_ws.ensure(home_bytes));
    size_t off = 0, nb = 0;
    MGPT_TRY(mgpt_moe_workspace_view(ep->home, n_tokens, "row_src", &off, &nb));
    const size_t row_cap = nb / sizeof(int32_t);
    MGPT_TRY(ep->rows.ensure(row_cap * rb));
    MGPT_TRY(ep->rows_back.ensure(row_cap * rb));
    MGPT_TRY(mgpt_moe_route_plan(ep->home, x, n_tokens, io, ep->home_ws.p, ep->home_ws.bytes, stream));
    MGPT_TRY(mgpt_moe_workspace_view(ep->home, n_tokens, "counts", &off, &nb));
    const int32_t* d_counts = (const int32_t*)((char*)ep->home_ws.p + off);

    // counts to the experts' owners: peer g gets, per chunk, my counts of its Ec experts; I get the peers' counts of mine
    MGPT_TRY(ep->recv_counts.ensure((size_t)G * nc * Ec * sizeof(int32_t)));
    int32_t* d_recv = (int32_t*)ep->recv_counts.p;          // [source][chunk][j]
    MGPT_TRY(follow(ep, st));
    // the rows are permuted while the counts travel and the host reads them
    MGPT_TRY(mgpt_moe_route_rows(ep->home, x, io, ep->home_ws.p, ep->home_ws.bytes, ep->rows.p, stream));
    if (G > 1) MGPT_NCCL(g_nccl.GroupStart());
    for (int c = 0; c < nc; ++c)
        for (int g = 0; g < G; ++g) {
            const int32_t* s = d_counts + (c * G + g) * Ec;
            int32_t* r = d_recv + (g * nc + c) * Ec;
            if (g == ep->rank) {
                MGPT_CUDA(cudaMemcpyAsync(r, s, Ec * sizeof(int32_t), cudaMemcpyDeviceToDevice, ep->cs));
            } else {
                MGPT_NCCL(g_nccl.Send(s, Ec * sizeof(int32_t), NCCL_BYTES, g, ep->comm, ep->cs));
                MGPT_NCCL(g_nccl.Recv(r, Ec * sizeof(int32_t), NCCL_BYTES, g, ep->comm, ep->cs));
            }
        }
    if (G > 1) MGPT_NCCL(g_nccl.GroupEnd());
    MGPT_CUDA(cudaMemcpyAsync(ep->h_counts, d_counts, (size_t)ep->E * sizeof(int32_t), cudaMemcpyDeviceToHost, ep->cs));
    MGPT_CUDA(cudaMemcpyAsync(ep->h_recv, d_recv, (size_t)G * nc * Ec * sizeof(int32_t), cudaMemcpyDeviceToHost, ep->cs));
    MGPT_CUDA(cudaStreamSynchronize(ep->cs));               // the one host synchronisation: how many rows go where

    ep->n_send = 0;
    for (int c = 0; c < nc; ++c) {
        ep->starts[c] = ep->n_send;
        for (int g = 0; g < G; ++g) {
            int s = 0, r = 0;
            for (int j = 0; j < Ec; ++j) {
                s += pad128(ep->h_counts[(c * G + g) * Ec + j]);
                r += pad128(ep->h_recv[(g * nc + c) * Ec + j]);
            }
            ep->send_split[c][g] = s;
            ep->recv_split[c][g] = r;
        }
        ep->n_send += sum(ep->send_split[c]);
        ep->n_recv[c] = sum(ep->recv_split[c]);
    }
    // buffers of the expert side (grown on demand), the real counts per (source, local expert) of each chunk
    for (int c = 0; c < nc; ++c) {
        const size_t bytes = (size_t)ep->n_recv[c] * rb;
        MGPT_TRY(ep->recv_rows[c].ensure(bytes));
        MGPT_TRY(ep->out_rows[c].ensure(bytes));
        MGPT_TRY(ep->local_ws[c].ensure(mgpt_moe_stage_workspace_bytes(ep->locals[c], ep->n_recv[c], 0)));
        MGPT_TRY(ep->seg_counts[c].ensure((size_t)G * Ec * sizeof(int32_t)));
        MGPT_CUDA(cudaMemcpy2DAsync(ep->seg_counts[c].p, Ec * sizeof(int32_t), d_recv + c * Ec, (size_t)nc * Ec * sizeof(int32_t),
                                    Ec * sizeof(int32_t), G, cudaMemcpyDeviceToDevice, ep->cs));
    }
    // every chunk's rows set off at once (they travel in this order); chunk c is computed while c+1 is arriving
    MGPT_TRY(follow(ep, st));                       // the permuted rows are complete
    for (int c = 0; c < nc; ++c) {
        MGPT_TRY(exchange_rows(ep, (char*)ep->recv_rows[c].p, ep->recv_split[c], (const char*)ep->rows.p + (size_t)ep->starts[c] * rb,
                               ep->send_split[c]));
        MGPT_CUDA(cudaEventRecord(ep->ev_in[c], ep->cs));
    }
    for (int c = 0; c < nc; ++c) {
        MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_in[c], 0));
        MGPT_TRY(mgpt_moe_experts_forward(ep->locals[c], ep->recv_rows[c].p, (const int32_t*)ep->seg_counts[c].p, G, ep->n_recv[c],
                                          ep->out_rows[c].p, ep->local_ws[c].p, ep->local_ws[c].bytes, stream));
        MGPT_CUDA(cudaEventRecord(ep->ev_out[c], st));
        MGPT_CUDA(cudaStreamWaitEvent(ep->cs, ep->ev_out[c], 0));
        MGPT_TRY(exchange_rows(ep, (char*)ep->rows_back.p + (size_t)ep->starts[c] * rb, ep->send_split[c],
                               (const char*)ep->out_rows[c].p, ep->recv_split[c]));
        MGPT_CUDA(cudaEventRecord(ep->ev_back[c], ep->cs));
    }
    for (int c = 0; c < nc; ++c) MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_back[c], 0));
    MGPT_TRY(mgpt_moe_combine(ep->home, ep->rows_back.p, y, io, ep->home_ws.p, ep->home_ws.bytes, stream));
    ep->last_n = n_tokens;
    ep->last_io = io;
    ep->fwd_done = true;
    return 0;
}

int mgpt_moe_ep_backward(mgpt_moe_ep* ep, const void* x, const void* dy, void* dx, int io, mgpt_stream_t stream)
{
    if (!ep) return fail(MGPT_MOE_EINVAL, "null argument");
    if (!ep->fwd_done) return fail(MGPT_MOE_ESTATE, "backward without a forward");
    if (io != ep->last_io) return fail(MGPT_MOE_ESTATE, "backward must use the forward's io dtype");
    if (!x || !dy || !dx) return fail(MGPT_MOE_EINVAL, "null token buffer");
    MGPT_CUDA(cudaSetDevice(ep->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const int nc = ep->nc;
    const size_t rb = (size_t)ep->C * ep->act;
    if (ep->peer) return backward_peer(ep, x, dy, dx, io, stream);
    MGPT_TRY(ep->d_rows.ensure(ep->rows.bytes));
    MGPT_TRY(ep->d_back.ensure(ep->rows.bytes));
    for (int c = 0; c < nc; ++c) {
        MGPT_TRY(ep->d_recv[c].ensure((size_t)ep->n_recv[c] * rb));
        MGPT_TRY(ep->d_in[c].ensure((size_t)ep->n_recv[c] * rb));
    }
    MGPT_TRY(mgpt_moe_combine_backward(ep->home, ep->rows_back.p, dy, io, ep->d_rows.p, ep->home_ws.p, ep->home_ws.bytes, stream));
    MGPT_TRY(follow(ep, st));
    for (int c = 0; c < nc; ++c) {
        MGPT_TRY(exchange_rows(ep, (char*)ep->d_recv[c].p, ep->recv_split[c], (const char*)ep->d_rows.p + (size_t)ep->starts[c] * rb,
                               ep->send_split[c]));
        MGPT_CUDA(cudaEventRecord(ep->ev_in[c], ep->cs));
    }
    for (int c = 0; c < nc; ++c) {
        MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_in[c], 0));
        // the rows' gradients first: they travel back while this chunk's parameter gradients are formed
        MGPT_TRY(mgpt_moe_experts_backward_rows(ep->locals[c], ep->d_recv[c].p, ep->d_in[c].p, ep->local_ws[c].p,
                                                ep->local_ws[c].bytes, stream));
        MGPT_CUDA(cudaEventRecord(ep->ev_out[c], st));
        MGPT_CUDA(cudaStreamWaitEvent(ep->cs, ep->ev_out[c], 0));
        MGPT_TRY(exchange_rows(ep, (char*)ep->d_back.p + (size_t)ep->starts[c] * rb, ep->send_split[c], (const char*)ep->d_in[c].p,
                               ep->recv_split[c]));
        MGPT_CUDA(cudaEventRecord(ep->ev_back[c], ep->cs));
        MGPT_TRY(mgpt_moe_experts_backward_params(ep->locals[c], ep->d_recv[c].p, ep->d_in[c].p, ep->local_ws[c].p,
                                                  ep->local_ws[c].bytes, stream));
    }
    for (int c = 0; c < nc; ++c) MGPT_CUDA(cudaStreamWaitEvent(st, ep->ev_back[c], 0));
    return mgpt_moe_route_backward(ep->home, x, ep->d_back.p, dx, io, ep->home_ws.p, ep->home_ws.bytes, stream);
}

}  // extern "C"
