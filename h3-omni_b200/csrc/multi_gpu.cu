// Host side of the library, part 3: everything that spans GPUs. NCCL communicators and the
// in-place Ulysses exchanges of the primitive ABI (reference cuda/h3_cuda.h:20-39,
// cuda/parallel.cuh:25-153), and the fused exchange over peer-memory windows (h3b_exchange_*).
#include <nccl.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "attn_kernels.h"
#include "h3_gpu_internal.h"

using h3b::bf16;
using h3b::cuda_good;
using h3b::fail;
using h3b::satisfied;

namespace h3b {
int rope_input(h3_gpu *g, QkvRopeInput &in, const h3_gpu_tensor *qkv, const h3_gpu_tensor *qn,
               const h3_gpu_tensor *kn, const h3_gpu_tensor *co, const h3_gpu_tensor *si, uint32_t rows,
               uint32_t heads, uint32_t dim, uint32_t half, float eps, int grouped);
}

// ======================= communicators =======================

struct h3_gpu_comm {
    ncclComm_t nccl;
    int rank, size;
};

// Message into a caller-supplied buffer (the calls below run before any context exists).
static int refuse(char *error, size_t size, const char *format, ...) {
    if (error && size) {
        va_list args;
        va_start(args, format);
        vsnprintf(error, size, format, args);
        va_end(args);
    }
    return 0;
}
static bool nccl_good(h3_gpu *g, ncclResult_t r, const char *what) {
    if (r != ncclSuccess) fail(g, "NCCL %s: %s", what, ncclGetErrorString(r));
    return r == ncclSuccess;
}

extern "C" int h3_gpu_device_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) count = 0;
    return count;
}
extern "C" int h3_gpu_select_device(int device, char *error, size_t size) {
    const cudaError_t e = cudaSetDevice(device);
    return e == cudaSuccess ? 1 : refuse(error, size, "cannot select CUDA device %d: %s", device, cudaGetErrorString(e));
}
// One process, one communicator per device 0..count-1 (the reference's rank threads, h3_dit.c:4066-4177).
extern "C" int h3_gpu_comm_init_all(int count, h3_gpu_comm **comms, char *error, size_t size) {
    if (count < 1 || count > 64 || !comms) return refuse(error, size, "invalid NCCL communicator count %d", count);
    std::vector<ncclComm_t> handles((size_t)count);
    const ncclResult_t r = ncclCommInitAll(handles.data(), count, nullptr);   // devices 0 .. count-1
    if (r != ncclSuccess) return refuse(error, size, "NCCL init: %s", ncclGetErrorString(r));
    for (int rank = 0; rank < count; rank++) comms[rank] = new h3_gpu_comm{handles[(size_t)rank], rank, count};
    return 1;
}
// One process per GPU: rank 0 makes the id, ships its 128 bytes by any transport, all ranks join.
extern "C" int h3b_comm_unique_id(void *id128, char *error, size_t size) {
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    if (!id128) return refuse(error, size, "NCCL unique id: no buffer");
    const ncclResult_t r = ncclGetUniqueId(static_cast<ncclUniqueId *>(id128));
    return r == ncclSuccess ? 1 : refuse(error, size, "NCCL unique id: %s", ncclGetErrorString(r));
}
extern "C" int h3b_comm_init_rank(const void *id128, int rank, int count, h3_gpu_comm **comm, char *error,
                                  size_t size) {
    if (!id128 || !comm || count < 1 || rank < 0 || rank >= count)
        return refuse(error, size, "invalid NCCL rank %d of %d", rank, count);
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    ncclComm_t handle;
    const ncclResult_t r = ncclCommInitRank(&handle, count, id, rank);
    if (r != ncclSuccess) return refuse(error, size, "NCCL init: %s", ncclGetErrorString(r));
    *comm = new h3_gpu_comm{handle, rank, count};
    return 1;
}
extern "C" int h3b_comm_rank(const h3_gpu_comm *c) { return c ? c->rank : -1; }
extern "C" int h3b_comm_size(const h3_gpu_comm *c) { return c ? c->size : 0; }
extern "C" void h3_gpu_comm_free(h3_gpu_comm *c) {
    if (c && c->nccl) ncclCommDestroy(c->nccl);
    delete c;
}
// After one rank has failed: ends the collectives the other ranks are waiting in. The
// communicator is unusable afterwards (every later call on it fails its argument check).
extern "C" void h3_gpu_comm_abort(h3_gpu_comm *c) {
    if (!c) return;
    ncclComm_t handle = c->nccl;
    c->nccl = nullptr;
    if (handle) ncclCommAbort(handle);
}

// ======================= Ulysses through NCCL (in place, with a scratch tensor) =======================

// Rank r's block p goes to rank p's block r. Peers are visited starting at the next rank, so the
// ranks do not all open with the same destination.
static bool all_to_all(h3_gpu *g, h3_gpu_comm *c, void *recv, const void *send, size_t block_bytes) {
    bool ok = nccl_good(g, ncclGroupStart(), "group start");
    for (int step = 0; ok && step < c->size; step++) {
        const int peer = (c->rank + 1 + step) % c->size;
        ok = nccl_good(g, ncclSend(static_cast<const char *>(send) + (size_t)peer * block_bytes, block_bytes, ncclUint8,
                                   peer, c->nccl, g->stream), "all-to-all send") &&
             nccl_good(g, ncclRecv(static_cast<char *>(recv) + (size_t)peer * block_bytes, block_bytes, ncclUint8, peer,
                                   c->nccl, g->stream), "all-to-all receive");
    }
    const ncclResult_t end = ncclGroupEnd();   // always closes the group that was opened
    return ok && nccl_good(g, end, "group end");
}

// scatter: [rows][heads][dim] on each rank -> [ranks*rows][heads/ranks][dim]: transpose the rank's
// tensor from [rows][ranks][group] to [ranks][rows][group] into the scratch, then exchange blocks.
// gather: the inverse: exchange blocks into the scratch, transpose back.
static int ulysses(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *t, h3_gpu_tensor *scratch, uint32_t rows, uint32_t heads,
                   uint32_t dim, bool scatter) {
    if (!g) return 0;
    if (!c || !c->nccl || heads % c->size) {
        fail(g, "Ulysses: %u heads do not split over %d ranks", heads, c ? c->size : 0);
        return 0;
    }
    const size_t count = (size_t)rows * heads * dim;
    if (!satisfied(g, {bf16(t, count, "Ulysses tensor"), bf16(scratch, count, "Ulysses scratch")})) return 0;
    const size_t group_bytes = (size_t)(heads / c->size) * dim * 2, block_bytes = (size_t)rows * group_bytes;
    if (group_bytes % 16) {
        fail(g, "Ulysses block of %zu bytes is not 16-byte aligned", group_bytes);
        return 0;
    }
    if (scatter)
        return cuda_good(g, h3b::transpose_rows_16b(scratch->data, t->data, rows, (unsigned)c->size, group_bytes / 16,
                                                    g->stream)) &&
               all_to_all(g, c, t->data, scratch->data, block_bytes);
    return all_to_all(g, c, scratch->data, t->data, block_bytes) &&
           cuda_good(g, h3b::transpose_rows_16b(t->data, scratch->data, (unsigned)c->size, rows, group_bytes / 16,
                                                g->stream));
}
extern "C" int h3_gpu_ulysses_scatter_heads_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *t, h3_gpu_tensor *scratch,
                                                 uint32_t rows, uint32_t heads, uint32_t dim) {
    return ulysses(g, c, t, scratch, rows, heads, dim, true);
}
extern "C" int h3_gpu_ulysses_gather_heads_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *t, h3_gpu_tensor *scratch,
                                                uint32_t rows, uint32_t heads, uint32_t dim) {
    return ulysses(g, c, t, scratch, rows, heads, dim, false);
}
// output[rank * count + i] = rank's input[i].
extern "C" int h3_gpu_all_gather_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                      size_t count) {
    if (!g || !c || !c->nccl) return 0;
    if (!satisfied(g, {bf16(input, count, "all-gather input"), bf16(output, count * (size_t)c->size, "all-gather output")}))
        return 0;
    return nccl_good(g, ncclAllGather(input->data, output->data, count * 2, ncclUint8, c->nccl, g->stream),
                     "all-gather");
}

// ======================= fused exchange over peer-memory windows =======================
// Each rank owns a window (one cudaMalloc) of `slots` tensors followed by a flag block. After
// connecting - through CUDA IPC handles when every rank is a process, or directly when the ranks
// are threads of one process - every rank holds pointers to all windows, and an exchange is one
// kernel (csrc/ulysses.cu) instead of a transpose kernel plus NCCL send/receive.
struct h3b_exchange {
    h3_gpu *gpu{};                       // null for an exchange made with h3b_exchange_create_raw
    int device{}, rank{}, ranks{}, slots{};
    size_t slot_elements{}, slot_bytes{}, flags_offset{};
    char *local{};                       // this rank's window
    char *mapped[h3b::EXCHANGE_MAX_RANKS]{};   // every rank's window as seen from here
    bool ipc_mapped[h3b::EXCHANGE_MAX_RANKS]{};
    unsigned long long epoch{}, limit_ns{2000000000ull};
    bool connected{};
    char error[256]{};
};

// Records the message in the exchange and, when it has one, in its context.
static cudaError_t exchange_error(h3b_exchange *x, cudaError_t code, const char *format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(x->error, sizeof x->error, format, args);
    va_end(args);
    if (x->gpu) fail(x->gpu, "%s", x->error);
    return code;
}
static cudaError_t exchange_cuda(h3b_exchange *x, cudaError_t e) {
    return e == cudaSuccess ? e : exchange_error(x, e, "CUDA: %s", cudaGetErrorString(e));
}
extern "C" const char *h3b_exchange_error(const h3b_exchange *x) { return x ? x->error : "no exchange"; }

extern "C" void h3b_exchange_free(h3b_exchange *x) {
    if (!x) return;
    if (x->gpu) cudaStreamSynchronize(x->gpu->stream);
    for (int p = 0; p < x->ranks; p++)
        if (x->ipc_mapped[p]) cudaIpcCloseMemHandle(x->mapped[p]);
    if (x->local) cudaFree(x->local);
    delete x;
}

extern "C" cudaError_t h3b_exchange_create_raw(int rank, int ranks, size_t slot_elements, int slots,
                                               h3b_exchange **exchange, void *handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!exchange || ranks < 1 || ranks > h3b::EXCHANGE_MAX_RANKS || rank < 0 || rank >= ranks || slots < 1 ||
        !slot_elements)
        return cudaErrorInvalidValue;
    auto *x = new (std::nothrow) h3b_exchange{};
    if (!x) return cudaErrorMemoryAllocation;
    x->rank = rank;
    x->ranks = ranks;
    x->slots = slots;
    x->slot_elements = slot_elements;
    x->slot_bytes = (slot_elements * 2 + 255) / 256 * 256;
    x->flags_offset = x->slot_bytes * (size_t)slots;
    const size_t bytes = x->flags_offset + sizeof(h3b::ExchangeFlags);
    cudaError_t e = cudaGetDevice(&x->device);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&x->local), bytes);
    if (e == cudaSuccess) e = cudaMemset(x->local, 0, bytes);
    if (e == cudaSuccess && handle64) {
        cudaIpcMemHandle_t handle;
        e = cudaIpcGetMemHandle(&handle, x->local);
        if (e == cudaSuccess) memcpy(handle64, &handle, 64);
    }
    if (e != cudaSuccess) {
        h3b_exchange_free(x);
        return e;
    }
    x->mapped[rank] = x->local;
    x->connected = ranks == 1;
    *exchange = x;
    return cudaSuccess;
}
extern "C" int h3b_exchange_create(h3_gpu *g, int rank, int ranks, size_t slot_elements, int slots,
                                   h3b_exchange **exchange, void *handle64) {
    if (!g || !exchange || !handle64) return 0;
    const cudaError_t e = h3b_exchange_create_raw(rank, ranks, slot_elements, slots, exchange, handle64);
    if (e == cudaErrorInvalidValue) {
        fail(g, "exchange: invalid rank %d of %d or empty window", rank, ranks);
        return 0;
    }
    if (!cuda_good(g, e)) return 0;
    (*exchange)->gpu = g;
    return 1;
}

// Ranks in separate processes. handles: ranks x 64 bytes in rank order (every rank's handle64,
// gathered by any transport).
extern "C" int h3b_exchange_connect(h3b_exchange *x, const void *handles) {
    if (!x || !handles) return 0;
    for (int p = 0; p < x->ranks; p++) {
        if (p == x->rank || x->mapped[p]) continue;
        cudaIpcMemHandle_t handle;
        memcpy(&handle, static_cast<const char *>(handles) + 64 * p, 64);
        void *mapped = nullptr;
        if (exchange_cuda(x, cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess)
            return 0;
        x->mapped[p] = static_cast<char *>(mapped);
        x->ipc_mapped[p] = true;
    }
    x->connected = true;
    return 1;
}

// Ranks as threads of ONE process (the reference's rank threads): an IPC handle cannot be opened
// by the process that made it, so the windows are joined by their plain device pointers, with
// peer access switched on between the devices. all_ranks: every rank's exchange in rank order;
// each rank calls this for its own exchange, with its own device current, after all ranks have
// created theirs.
extern "C" int h3b_exchange_connect_local(h3b_exchange *x, h3b_exchange *const *all_ranks) {
    if (!x || !all_ranks) return 0;
    for (int p = 0; p < x->ranks; p++) {
        const h3b_exchange *peer = all_ranks[p];
        if (!peer || peer->ranks != x->ranks || peer->rank != p || peer->slot_bytes != x->slot_bytes ||
            peer->slots != x->slots) {
            exchange_error(x, cudaErrorInvalidValue, "exchange: rank %d of the local group does not match", p);
            return 0;
        }
        if (peer->device != x->device) {
            const cudaError_t e = cudaDeviceEnablePeerAccess(peer->device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) {
                cudaGetLastError();   // not an error: clear it
            } else if (exchange_cuda(x, e) != cudaSuccess) {
                return 0;
            }
        }
        x->mapped[p] = peer->local;
    }
    x->connected = true;
    return 1;
}

// Bound of every device-side wait of this exchange's kernels (default 2000 ms).
extern "C" int h3b_exchange_set_wait_limit_ms(h3b_exchange *x, unsigned milliseconds) {
    if (!x || !milliseconds) return 0;
    x->limit_ns = (unsigned long long)milliseconds * 1000000ull;
    return 1;
}

extern "C" void *h3b_exchange_slot_pointer(h3b_exchange *x, int slot) {
    return x && slot >= 0 && slot < x->slots ? x->local + x->slot_bytes * (size_t)slot : nullptr;
}
// Non-owning tensor over slot `slot` of this rank's window (free it with h3_gpu_tensor_free).
extern "C" h3_gpu_tensor *h3b_exchange_slot(h3b_exchange *x, int slot) {
    void *p = h3b_exchange_slot_pointer(x, slot);
    return p && x->gpu ? h3b_tensor_wrap(x->gpu, p, x->slot_elements, H3_GPU_BF16) : nullptr;
}

// The synchronisation block of the next exchange (takes the next epoch).
static cudaError_t next_sync(h3b_exchange *x, h3b::ExchangeSync &sync) {
    if (!x->connected) return exchange_error(x, cudaErrorInvalidValue, "exchange: not connected");
    int current = -1;
    cudaError_t e = cudaGetDevice(&current);
    if (e == cudaSuccess && current != x->device)
        return exchange_error(x, cudaErrorInvalidDevice, "exchange of device %d used while device %d is current",
                              x->device, current);
    if (e == cudaSuccess) e = h3b::device_status_word(&sync.status);
    if (e != cudaSuccess) return exchange_cuda(x, e);
    for (int p = 0; p < x->ranks; p++)
        sync.flags[p] = reinterpret_cast<h3b::ExchangeFlags *>(x->mapped[p] + x->flags_offset);
    sync.epoch = ++x->epoch;
    sync.limit_ns = x->limit_ns;
    sync.rank = x->rank;
    sync.ranks = x->ranks;
    return cudaSuccess;
}

static cudaError_t push(h3b_exchange *x, bool gather, int count, const int *slots, const void *const *sources,
                        uint32_t rows, uint32_t heads, uint32_t dim, cudaStream_t stream) {
    if (!x) return cudaErrorInvalidValue;
    if (count < 1 || count > h3b::EXCHANGE_MAX_TENSORS || !slots || !sources)
        return exchange_error(x, cudaErrorInvalidValue, "exchange: 1 to %d tensors per call", h3b::EXCHANGE_MAX_TENSORS);
    const size_t elements = (size_t)rows * heads * dim;
    if (!rows || !heads || heads % x->ranks || (dim * 2) % 16 || elements > x->slot_elements)
        return exchange_error(x, cudaErrorInvalidValue,
                              "exchange: %u heads over %d ranks, or %zu elements exceed the slot of %zu", heads,
                              x->ranks, elements, x->slot_elements);
    void *window[h3b::EXCHANGE_MAX_TENSORS][h3b::EXCHANGE_MAX_RANKS];
    for (int t = 0; t < count; t++) {
        bool bad = slots[t] < 0 || slots[t] >= x->slots || !sources[t];
        for (int o = 0; o < t; o++) bad = bad || slots[o] == slots[t];
        if (bad) return exchange_error(x, cudaErrorInvalidValue, "exchange: bad or repeated slot %d", slots[t]);
        for (int p = 0; p < x->ranks; p++)
            window[t][p] = x->mapped[p] ? x->mapped[p] + x->slot_bytes * (size_t)slots[t] : nullptr;
    }
    h3b::ExchangeSync sync{};
    const cudaError_t e = next_sync(x, sync);
    if (e != cudaSuccess) return e;
    return exchange_cuda(x, h3b::exchange_push(gather, count, sources, window, sync, rows, heads, dim, stream));
}
extern "C" cudaError_t h3b_exchange_scatter_raw(h3b_exchange *x, int count, const int *slots,
                                                const void *const *sources, uint32_t rows, uint32_t heads,
                                                uint32_t dim, cudaStream_t stream) {
    return push(x, false, count, slots, sources, rows, heads, dim, stream);
}
extern "C" cudaError_t h3b_exchange_gather_raw(h3b_exchange *x, int slot, const void *source, uint32_t rows,
                                               uint32_t heads, uint32_t dim, cudaStream_t stream) {
    return push(x, true, 1, &slot, &source, rows, heads, dim, stream);
}

// The same on tensors of the exchange's context, on the context's stream.
static int push_tensors(h3b_exchange *x, bool gather, int count, const int *slots, const h3_gpu_tensor *const *sources,
                        uint32_t rows, uint32_t heads, uint32_t dim) {
    if (!x || !x->gpu) return 0;
    if (count < 1 || count > h3b::EXCHANGE_MAX_TENSORS || !sources) {
        fail(x->gpu, "exchange: 1 to %d tensors per call", h3b::EXCHANGE_MAX_TENSORS);
        return 0;
    }
    const void *raw[h3b::EXCHANGE_MAX_TENSORS];
    for (int t = 0; t < count; t++) {
        if (!satisfied(x->gpu, {bf16(sources[t], (size_t)rows * heads * dim, "exchange source")})) return 0;
        raw[t] = sources[t]->data;
    }
    return push(x, gather, count, slots, raw, rows, heads, dim, x->gpu->stream) == cudaSuccess;
}
// src [rows][heads][dim] on each rank -> slot of every rank: [ranks*rows][heads/ranks][dim].
extern "C" int h3b_exchange_scatter_heads_bf16(h3b_exchange *x, int slot, const h3_gpu_tensor *src, uint32_t rows,
                                               uint32_t heads, uint32_t dim) {
    return push_tensors(x, false, 1, &slot, &src, rows, heads, dim);
}
// Up to four tensors of one shape (q, k, v, gate ...) in ONE kernel and one pair of handshakes.
extern "C" int h3b_exchange_scatter_heads_multi_bf16(h3b_exchange *x, int count, const int *slots,
                                                     const h3_gpu_tensor *const *sources, uint32_t rows,
                                                     uint32_t heads, uint32_t dim) {
    return push_tensors(x, false, count, slots, sources, rows, heads, dim);
}
// src [ranks*rows][heads/ranks][dim] on each rank -> slot of every rank: [rows][heads][dim].
extern "C" int h3b_exchange_gather_heads_bf16(h3b_exchange *x, int slot, const h3_gpu_tensor *src, uint32_t rows,
                                              uint32_t heads, uint32_t dim) {
    return push_tensors(x, true, 1, &slot, &src, rows, heads, dim);
}

// Attention with the sequence-gather fused into its epilogue: every rank attends all `sequence`
// rows for its heads / ranks heads (q, k, v: [>= sequence][heads/ranks][128], e.g. the scatter
// slots) and each finished output row is stored straight into the row shard of the rank that owns
// it, slot `slot` of that rank's window laid out [rows][heads][128]. Open (the owners have
// stopped reading the slot), attention, close (all rows have arrived).
extern "C" int h3b_exchange_sdpa_gather_bf16(h3b_exchange *x, int slot, const h3_gpu_tensor *q,
                                             const h3_gpu_tensor *k, const h3_gpu_tensor *v, uint32_t sequence,
                                             uint32_t rows, uint32_t heads, float scale) {
    if (!x || !x->gpu) return 0;
    h3_gpu *g = x->gpu;
    if (!x->connected || slot < 0 || slot >= x->slots || !heads || heads % x->ranks || !rows ||
        (size_t)rows * heads * 128 > x->slot_elements || (size_t)sequence > (size_t)rows * x->ranks) {
        fail(g, "fused attention+gather: not connected, bad slot or shape (%u rows x %d ranks, %u heads)", rows,
             x->ranks, heads);
        return 0;
    }
    const uint32_t local_heads = heads / x->ranks;
    const size_t need = (size_t)sequence * local_heads * 128;
    if (!satisfied(g, {bf16(q, need, "attention query"), bf16(k, need, "attention key"),
                       bf16(v, need, "attention value")}))
        return 0;
    h3b::PeerOutput peer{};
    for (int p = 0; p < x->ranks; p++) peer.base[p] = x->mapped[p] + x->slot_bytes * (size_t)slot;
    peer.rows_per_rank = rows;
    peer.rank = (unsigned)x->rank;
    peer.total_heads = heads;
    h3b::ExchangeSync sync{};
    if (next_sync(x, sync) != cudaSuccess) return 0;
    return cuda_good(g, h3b::exchange_open(sync, g->stream)) &&
           cuda_good(g, h3b::attn_dense_tc5(nullptr, q->data, k->data, v->data, nullptr, 1, sequence, sequence,
                                            local_heads, local_heads, scale, g->stream, &peer)) &&
           cuda_good(g, h3b::exchange_close(sync, g->stream));
}

// Producer fused with the head scatter: norm + rotation store each (row, head) vector of q, k
// and v into the owning rank's slots; open, kernel, close.
extern "C" int h3b_exchange_qkv_rope_scatter_bf16(h3b_exchange *x, int slot_q, int slot_k, int slot_v,
                                                  const h3_gpu_tensor *qkv, const h3_gpu_tensor *qn,
                                                  const h3_gpu_tensor *kn, const h3_gpu_tensor *co,
                                                  const h3_gpu_tensor *si, uint32_t rows, uint32_t heads,
                                                  uint32_t rope_half, float eps, int grouped) {
    if (!x || !x->gpu) return 0;
    h3_gpu *g = x->gpu;
    const int slots[3] = {slot_q, slot_k, slot_v};
    bool bad = !x->connected || !heads || heads % x->ranks || (size_t)rows * heads * 128 > x->slot_elements;
    for (int t = 0; t < 3; t++) {
        bad = bad || slots[t] < 0 || slots[t] >= x->slots;
        for (int o = 0; o < t; o++) bad = bad || slots[t] == slots[o];
    }
    if (bad) {
        fail(g, "fused norm/RoPE scatter: not connected, bad slots or shape (%u rows, %u heads, %d ranks)", rows, heads,
             x->ranks);
        return 0;
    }
    h3b::QkvRopeInput in{};
    if (!h3b::rope_input(g, in, qkv, qn, kn, co, si, rows, heads, 128, rope_half, eps, grouped)) return 0;
    void *window[3][h3b::EXCHANGE_MAX_RANKS];
    for (int p = 0; p < x->ranks; p++)
        for (int t = 0; t < 3; t++) window[t][p] = x->mapped[p] + x->slot_bytes * (size_t)slots[t];
    h3b::ExchangeSync sync{};
    if (next_sync(x, sync) != cudaSuccess) return 0;
    return cuda_good(g, h3b::exchange_open(sync, g->stream)) &&
           cuda_good(g, h3b::qkv_rope_head_shards(in, window[0], window[1], window[2], x->rank, x->ranks, g->stream)) &&
           cuda_good(g, h3b::exchange_close(sync, g->stream));
}
