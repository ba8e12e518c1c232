// Row-sharded CSR SpMM across the GPUs of one node: one process per GPU, each holding a block of rows of A
// (and of C) and the rows of B of the vertices it owns.  A product needs rows of B that other ranks own, so
// every product is: pack the rows the others need -> exchange over NCCL (NVLink / NVSwitch) into this GPU's
// own memory -> local product.  The reference is single-GPU (test/test_all.cpp:27-109 is one process on one
// device) and has no counterpart.
//
// What crosses NVLink.  A shard references only part of B: on a power-law graph split eight ways a shard
// touches a fifth of the rows, and on any graph the rows of isolated vertices are never read.  The plan
// therefore lists, per owner, the rows this shard's column indices name, renumbers the shard's columns into
// that compact list (owner after owner, ascending inside an owner), and tells every owner which of its rows
// to send here.  A product then moves exactly the referenced rows, each once, and the local kernel reads a
// dense n_needed x K matrix.  HPSPMM_EXCHANGE_ALL_ROWS keeps the plain all-gather (every row to everybody)
// for comparison and for callers that need the whole of B afterwards.
//
// Overlap.  The exchange runs on the plan's own stream, the product on the caller's.  begin() only needs
// B_own; product() only needs the exchange of its slot.  A caller with several independent products (the
// layers of a model that are evaluated together, or the K = 32 / 64 / 128 products of the benchmark) begins
// them all and then multiplies them in turn: while one slot multiplies, the next slot's rows are in flight.
//
// Transport.  By default the rows are PUSHED: one kernel per exchange reads the rows the other ranks need
// from B_own and stores them straight into the receivers' dense operands through peer mappings of those
// buffers (CUDA IPC, plain stores over NVLink / NVSwitch, every SM taking part), the own referenced rows
// going to the local operand by the same launch; no send buffer, no second copy.  A four-byte NCCL
// all-reduce behind the kernel is the completion signal: when it has finished on a rank, every rank's push
// kernel has, and a kernel's stores are visible once it has ended.  Every slot holds two operand buffers used
// in turn, and a rank joins a slot's next signal only after its own last product on that slot has read its
// buffer, so a push never overtakes the product that still reads its target.  With
// HPSPMM_EXCHANGE_NEEDED_ROWS_NCCL (or when a peer mapping cannot be had) the rows are packed into a send
// buffer and travel by grouped ncclSend / ncclRecv instead; measured on two B200s that path moves 0.36 TB/s
// per direction, the push 0.6 TB/s or more.  No TMA and no multicast anywhere in this file.
//
// NCCL is looked up at run time (dlopen of libnccl.so.2; the copy a host framework has already loaded is
// reused), so the library itself links against nothing but the CUDA runtime and single-GPU users need no
// NCCL at all.  No kernel of this file READS another GPU's memory (each row of B is gathered many times, so
// remote rows always land in local HBM first), and there is no device-side wait anywhere: ordering is by
// stream events and by the completion of NCCL operations.
#include <dlfcn.h>
#include <stdlib.h>

#include <algorithm>
#include <mutex>
#include <new>
#include <vector>

#include "hpspmm_internal.h"

namespace {

// ---- the few NCCL entry points used, bound by name -------------------------------------------------
struct nccl_id {
  char internal[128];
};
typedef void* nccl_comm_t;
constexpr int kNcclInt32 = 2;    // ncclInt32
constexpr int kNcclFloat32 = 7;  // ncclFloat32
constexpr int kNcclUint8 = 1;    // ncclUint8
constexpr int kNcclSum = 0;      // ncclSum
constexpr int kMaxPushWorld = 16;

struct nccl_api {
  void* handle;
  int (*GetUniqueId)(nccl_id*);
  int (*CommInitRank)(nccl_comm_t*, int, nccl_id, int);
  int (*CommDestroy)(nccl_comm_t);
  int (*Send)(const void*, size_t, int, int, nccl_comm_t, cudaStream_t);
  int (*Recv)(void*, size_t, int, int, nccl_comm_t, cudaStream_t);
  int (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t);
  int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t);
  int (*GroupStart)();
  int (*GroupEnd)();
  const char* (*GetErrorString)(int);
};

nccl_api g_nccl;
std::mutex g_nccl_mutex;

const nccl_api* load_nccl(char* err, size_t err_len) {
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.handle) return &g_nccl;
  // the copy the process already holds (a framework's), else whatever the loader finds
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    if (err && err_len) snprintf(err, err_len, "NCCL not found: %s", dlerror());
    return nullptr;
  }
  nccl_api api;
  memset(&api, 0, sizeof(api));
  api.handle = h;
#define HPSPMM_BIND(field, name)                                       \
  api.field = reinterpret_cast<decltype(api.field)>(dlsym(h, name));   \
  if (!api.field) {                                                    \
    if (err && err_len) snprintf(err, err_len, "NCCL lacks %s", name); \
    return nullptr;                                                    \
  }
  HPSPMM_BIND(GetUniqueId, "ncclGetUniqueId")
  HPSPMM_BIND(CommInitRank, "ncclCommInitRank")
  HPSPMM_BIND(CommDestroy, "ncclCommDestroy")
  HPSPMM_BIND(Send, "ncclSend")
  HPSPMM_BIND(Recv, "ncclRecv")
  HPSPMM_BIND(AllGather, "ncclAllGather")
  HPSPMM_BIND(AllReduce, "ncclAllReduce")
  HPSPMM_BIND(GroupStart, "ncclGroupStart")
  HPSPMM_BIND(GroupEnd, "ncclGroupEnd")
  HPSPMM_BIND(GetErrorString, "ncclGetErrorString")
#undef HPSPMM_BIND
  g_nccl = api;
  return &g_nccl;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__global__ void rebase_rows_kernel(int* __restrict__ rows, int64_t n, int base) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) rows[i] -= base;
}

constexpr int kSlots = 4;

// Where the rows of one exchange go: destination after destination in the order of the send list
// (the other ranks ascending, then this rank itself).
struct push_targets {
  float* base[kMaxPushWorld];      // receiver's dense operand (a peer mapping, or the local buffer)
  int64_t first_row[kMaxPushWorld];   // row of that operand where this rank's block starts
  int64_t list_begin[kMaxPushWorld + 1];   // positions in the send list
  int n;
};

// dst_d[first_row_d + i - list_begin_d, :] = B_own[send_rows[i], :] for every position i of the send list;
// one 16-byte (VEC = 4) or 4-byte element per thread step, rows written whole and in order, so the
// stores that cross NVLink are contiguous runs of K * 4 bytes.
constexpr int kPushThreads = 64;   // the product kernels' block size: a push block fits the slot a product block leaves

template <int VEC>
__global__ void __launch_bounds__(kPushThreads)
push_rows_kernel(const float* __restrict__ B_own, const int* __restrict__ send_rows, int64_t total_rows,
                 int64_t row_elems, push_targets t) {
  constexpr int UNROLL = 4;   // independent load -> remote store pairs in flight per thread
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t total = total_rows * row_elems;
  for (int64_t e0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e0 < total; e0 += stride * UNROLL) {
    float4 v4[UNROLL];
    float v1[UNROLL];
    int64_t dst[UNROLL];
    int dd[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t e = e0 + u * stride;
      dd[u] = -1;
      if (e < total) {
        const int64_t i = e / row_elems, c = e - i * row_elems;
        int d = 0;
#pragma unroll 1
        while (d + 1 < t.n && i >= t.list_begin[d + 1]) ++d;
        const int64_t src = (int64_t)__ldg(send_rows + i) * row_elems + c;
        dst[u] = (t.first_row[d] + (i - t.list_begin[d])) * row_elems + c;
        dd[u] = d;
        if (VEC == 4)
          v4[u] = __ldg(reinterpret_cast<const float4*>(B_own) + src);
        else
          v1[u] = __ldg(B_own + src);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (dd[u] < 0) continue;
      if (VEC == 4)
        reinterpret_cast<float4*>(t.base[dd[u]])[dst[u]] = v4[u];
      else
        t.base[dd[u]][dst[u]] = v1[u];
    }
  }
}

}  // namespace

struct hpspmm_comm {
  int device;
  int world, rank;
  nccl_comm_t comm;
  const nccl_api* api;
};

struct hpspmm_shard_slot {
  int64_t K_cap;        // width the buffers and the plan were sized for (0 = unused)
  float* send_buf;      // NCCL transport: rows for the other ranks, destination after destination
  float* B_local[2];    // the n_needed x K matrix the product reads; push transport: two, used in turn
  float* peer[2][kMaxPushWorld];   // push transport: the other ranks' B_local buffers, mapped here
  int phase;            // which of the two buffers the last begin filled
  bool begun;           // an exchange has been begun and its product not yet enqueued
  hpspmm_plan* plan;    // chunk table of the shard for this width class
  cudaEvent_t ev_in, ev_landed, ev_read;
  bool read_pending;    // a product of this slot has been enqueued since the last begin
};

struct hpspmm_shard_plan {
  int device;
  int world, rank;
  hpspmm_comm* comm;
  int exchange;
  int64_t M_local, N, nnz_local, n_needed, max_K;
  int64_t rows_own;                  // rows of B this rank owns
  std::vector<int64_t> recv_off;     // world + 1: where owner s's rows start in B_local
  std::vector<int64_t> send_cnt;     // world: rows this rank sends to d (send_cnt[rank] = own rows it needs)
  std::vector<int64_t> send_off;     // world + 1 offsets into send_rows, order: d != rank ascending, then rank
  int64_t send_remote;               // rows sent to other ranks
  int32_t* d_row_ptr;                // shard's row_ptr (M_local + 1)
  int32_t* d_col;                    // shard's columns renumbered into B_local's rows
  int32_t* d_send_rows;              // local row ids of B_own, grouped as send_off says
  cudaStream_t comm_stream;
  bool push;                         // rows travel by peer stores (else by NCCL send / receive)
  int64_t push_blocks;               // grid of the push kernel (64-thread blocks)
  std::vector<int64_t> dst_first_row;   // world: where this rank's block starts in rank d's dense operand
  int32_t* d_token;                  // four bytes for the completion signal
  hpspmm_shard_slot slots[kSlots];
  size_t device_bytes;
};

namespace {

int nccl_fail(hpspmm_ctx* ctx, const nccl_api* api, const char* what, int rc) {
  if (ctx) snprintf(ctx->err, sizeof(ctx->err), "%s: NCCL error %d (%s)", what, rc, api ? api->GetErrorString(rc) : "?");
  return HPSPMM_ERR_CUDA;
}

#define HPSPMM_NCCL_TRY(ctx, api, call)                         \
  do {                                                          \
    const int rc__ = (call);                                    \
    if (rc__ != 0) return nccl_fail((ctx), (api), #call, rc__); \
  } while (0)

// position of destination d in the send order (others ascending, self last)
inline int send_slot_of(int d, int rank, int world) { return d == rank ? world - 1 : (d < rank ? d : d - 1); }

// Unmaps the other ranks' buffers of a slot; true if there was anything to unmap.
bool close_peer_mappings(hpspmm_shard_slot& s) {
  bool any = false;
  for (int b = 0; b < 2; ++b)
    for (int d = 0; d < kMaxPushWorld; ++d)
      if (s.peer[b][d]) {
        cudaIpcCloseMemHandle(s.peer[b][d]);
        s.peer[b][d] = nullptr;
        any = true;
      }
  return any;
}

// All ranks meet here (the four-byte all-reduce, waited for on the host).  An exported buffer must not be freed
// while another process still has it mapped, so buffers are released in two steps: every rank unmaps what it
// had mapped, the ranks meet, and only then does each free its own.
void meet_all_ranks(hpspmm_shard_plan* p) {
  if (p->world <= 1 || !p->comm || !p->comm->comm || !p->d_token || !p->comm_stream) return;
  const nccl_api* api = p->comm->api;
  if (api->AllReduce(p->d_token, p->d_token + 1, 1, kNcclInt32, kNcclSum, p->comm->comm, p->comm_stream) == 0)
    cudaStreamSynchronize(p->comm_stream);
}

// Collective: true on every rank iff `ok` was true on every rank.  Used in set-up paths so that a failure on
// one rank (an allocation, a mapping) makes all ranks return an error instead of leaving the others inside a
// collective the failed rank never joins.
bool all_ranks_ok(hpspmm_shard_plan* p, bool ok, cudaStream_t stream) {
  if (p->world <= 1 || !p->comm || !p->comm->comm || !p->d_token) return ok;
  const nccl_api* api = p->comm->api;
  int32_t bad = ok ? 0 : 1, total = 1;
  int32_t* cell = p->d_token + 8;
  if (cudaMemcpyAsync(cell, &bad, 4, cudaMemcpyHostToDevice, stream) != cudaSuccess) return false;
  if (api->AllReduce(cell, cell + 1, 1, kNcclInt32, kNcclSum, p->comm->comm, stream) != 0) return false;
  if (cudaMemcpyAsync(&total, cell + 1, 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return false;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return false;
  return total == 0;
}

void release_slot_buffers(hpspmm_ctx* ctx, hpspmm_shard_plan* p, hpspmm_shard_slot& s) {
  if (close_peer_mappings(s)) meet_all_ranks(p);
  for (int b = 0; b < 2; ++b) {
    if (s.B_local[b]) cudaFree(s.B_local[b]);
    s.B_local[b] = nullptr;
  }
  if (s.send_buf) cudaFree(s.send_buf);
  s.send_buf = nullptr;
  if (s.plan) hpspmm_plan_destroy(ctx, s.plan);
  s.plan = nullptr;
  s.K_cap = 0;
}

// First use of a slot at this width (or a wider one): allocate the operand buffers, build the chunk table and,
// for the push transport, map every other rank's buffers.  Collective when world > 1; synchronises.
int ensure_slot(hpspmm_ctx* ctx, hpspmm_shard_plan* p, int slot, int64_t K, cudaStream_t user_stream) {
  hpspmm_shard_slot& s = p->slots[slot];
  // (a plan that has fallen back to the NCCL transport rebuilds the slots that were set up for the push)
  if (s.K_cap >= K && s.plan != nullptr && (p->push || s.send_buf != nullptr || p->world == 1)) return HPSPMM_OK;
  HPSPMM_CUDA_TRY(ctx, cudaDeviceSynchronize());
  release_slot_buffers(ctx, p, s);
  const int world = p->world, rank = p->rank;
  const int n_buf = p->push ? 2 : 1;
  const size_t b_loc = align_up((size_t)std::max<int64_t>(p->n_needed, 1) * (size_t)K * 4, 256);
  cudaError_t ea = cudaSuccess;
  for (int b = 0; b < n_buf && ea == cudaSuccess; ++b) {
    ea = hpspmm_device_malloc((void**)&s.B_local[b], b_loc);
    if (ea == cudaSuccess) p->device_bytes += b_loc;
  }
  if (!p->push && ea == cudaSuccess) {
    const size_t b_send = align_up((size_t)std::max<int64_t>(p->send_remote, 1) * (size_t)K * 4, 256);
    ea = hpspmm_device_malloc((void**)&s.send_buf, b_send);
    if (ea == cudaSuccess) p->device_bytes += b_send;
  }
  if (ea == cudaSuccess && !s.ev_in) {
    ea = cudaEventCreateWithFlags(&s.ev_in, cudaEventDisableTiming);
    if (ea == cudaSuccess) ea = cudaEventCreateWithFlags(&s.ev_landed, cudaEventDisableTiming);
    if (ea == cudaSuccess) ea = cudaEventCreateWithFlags(&s.ev_read, cudaEventDisableTiming);
  }
  // every rank learns whether every rank got its buffers before any of them enters the handle exchange
  if (!all_ranks_ok(p, ea == cudaSuccess, user_stream)) {
    release_slot_buffers(ctx, p, s);
    if (ea != cudaSuccess)
      return hpspmm_set_err(ctx, ea == cudaErrorMemoryAllocation ? HPSPMM_ERR_OOM : HPSPMM_ERR_CUDA, "slot buffers", ea);
    snprintf(ctx->err, sizeof(ctx->err), "another rank could not allocate its slot buffers");
    return HPSPMM_ERR_OOM;
  }
  if (p->push && world > 1) {
    // every rank publishes the handles of its two buffers; all ranks map all of them
    const nccl_api* api = p->comm->api;
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    std::vector<unsigned char> mine(2 * hb), all((size_t)world * 2 * hb);
    for (int b = 0; b < 2; ++b) {
      cudaIpcMemHandle_t h;
      HPSPMM_CUDA_TRY(ctx, cudaIpcGetMemHandle(&h, s.B_local[b]));
      memcpy(mine.data() + b * hb, &h, hb);
    }
    unsigned char* d_h = nullptr;
    HPSPMM_CUDA_TRY(ctx, hpspmm_device_malloc((void**)&d_h, (size_t)(world + 1) * 2 * hb));
    cudaError_t e = cudaMemcpyAsync(d_h, mine.data(), 2 * hb, cudaMemcpyHostToDevice, user_stream);
    int rc = 0;
    if (e == cudaSuccess) rc = api->AllGather(d_h, d_h + 2 * hb, 2 * hb, kNcclUint8, p->comm->comm, user_stream);
    if (e == cudaSuccess && rc == 0)
      e = cudaMemcpyAsync(all.data(), d_h + 2 * hb, (size_t)world * 2 * hb, cudaMemcpyDeviceToHost, user_stream);
    if (e == cudaSuccess && rc == 0) e = cudaStreamSynchronize(user_stream);
    cudaFree(d_h);
    if (rc != 0) return nccl_fail(ctx, api, "ncclAllGather(buffer handles)", rc);
    if (e != cudaSuccess) return hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "buffer handle exchange", e);
    for (int d = 0; d < world && e == cudaSuccess; ++d) {
      if (d == rank) continue;
      for (int b = 0; b < 2 && e == cudaSuccess; ++b) {
        cudaIpcMemHandle_t h;
        memcpy(&h, all.data() + ((size_t)d * 2 + b) * hb, hb);
        void* ptr = nullptr;
        e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) s.peer[b][d] = (float*)ptr;
      }
    }
    // test seam: HPSPMM_DEBUG_FAIL_PEER_MAPPING=<rank> makes that rank behave as if a mapping had failed
    if (const char* env = getenv("HPSPMM_DEBUG_FAIL_PEER_MAPPING"))
      if (atoi(env) == rank && e == cudaSuccess) e = cudaErrorInvalidDevice;
    if (!all_ranks_ok(p, e == cudaSuccess, user_stream)) {
      // Some rank cannot map a peer's buffer (no peer access between two of the devices, IPC not permitted in
      // this process ...).  Every rank has just learnt it, so all of them fall back together to the transport that
      // needs no mapping: the same rows, packed and sent with ncclSend / ncclRecv.
      close_peer_mappings(s);   // whatever this rank had mapped; then every rank meets before anybody frees
      meet_all_ranks(p);
      release_slot_buffers(ctx, p, s);
      if (e != cudaSuccess) cudaGetLastError();   // the failed mapping is not an error of this call
      p->push = false;
      return ensure_slot(ctx, p, slot, K, user_stream);
    }
  }
  int st = hpspmm_plan_create(ctx, p->M_local, p->n_needed, p->nnz_local, p->d_row_ptr, p->d_col, K, nullptr,
                              (hpspmm_stream)user_stream, &s.plan);
  if (st != HPSPMM_OK) return st;
  s.K_cap = K;
  s.read_pending = false;
  s.begun = false;
  s.phase = 0;
  return HPSPMM_OK;
}

}  // namespace

extern "C" {

int hpspmm_comm_unique_id(unsigned char* id_out) {
  if (!id_out) return HPSPMM_ERR_INVALID;
  const nccl_api* api = load_nccl(nullptr, 0);
  if (!api) return HPSPMM_ERR_UNSUPPORTED;
  nccl_id id;
  if (api->GetUniqueId(&id) != 0) return HPSPMM_ERR_CUDA;
  memcpy(id_out, id.internal, sizeof(id.internal));
  return HPSPMM_OK;
}

int hpspmm_comm_create(hpspmm_ctx* ctx, int32_t world, int32_t rank, const unsigned char* id, hpspmm_comm** out) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr && out != nullptr, "null context or output");
  *out = nullptr;
  HPSPMM_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world, "bad world size or rank");
  hpspmm_comm* c = new (std::nothrow) hpspmm_comm();
  if (!c) return HPSPMM_ERR_OOM;
  c->device = ctx->device;
  c->world = world;
  c->rank = rank;
  c->comm = nullptr;
  c->api = nullptr;
  if (world > 1) {
    if (!id) {
      delete c;
      HPSPMM_REQUIRE(ctx, false, "null communicator id");
    }
    c->api = load_nccl(ctx->err, sizeof(ctx->err));
    if (!c->api) {
      delete c;
      return HPSPMM_ERR_UNSUPPORTED;
    }
    hpspmm_device_guard guard(ctx->device);
    nccl_id nid;
    memcpy(nid.internal, id, sizeof(nid.internal));
    const int rc = c->api->CommInitRank(&c->comm, world, nid, rank);
    if (rc != 0) {
      const nccl_api* api = c->api;
      delete c;
      return nccl_fail(ctx, api, "ncclCommInitRank", rc);
    }
  }
  *out = c;
  return HPSPMM_OK;
}

int hpspmm_comm_destroy(hpspmm_comm* comm) {
  if (!comm) return HPSPMM_OK;
  if (comm->comm && comm->api) {
    hpspmm_device_guard guard(comm->device);
    comm->api->CommDestroy(comm->comm);
  }
  delete comm;
  return HPSPMM_OK;
}

int hpspmm_comm_info(const hpspmm_comm* comm, int32_t* world, int32_t* rank) {
  if (!comm) return HPSPMM_ERR_INVALID;
  if (world) *world = comm->world;
  if (rank) *rank = comm->rank;
  return HPSPMM_OK;
}

int hpspmm_shard_plan_create(hpspmm_ctx* ctx, hpspmm_comm* comm, int64_t M_local, int64_t N, int64_t nnz_local,
                             const int32_t* row_ptr_host, const int32_t* col_idx_host, const int64_t* b_bounds,
                             int64_t max_K, int32_t exchange, hpspmm_stream stream, hpspmm_shard_plan** out) {
  HPSPMM_TRACE("hpspmm_shard_plan_create");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && out != nullptr, "null context or output");
  *out = nullptr;
  HPSPMM_REQUIRE(ctx, comm != nullptr && comm->device == ctx->device, "communicator missing or on another device");
  HPSPMM_REQUIRE(ctx, M_local >= 0 && N >= 1 && nnz_local >= 0 && max_K >= 1, "bad size");
  HPSPMM_REQUIRE(ctx, row_ptr_host != nullptr && (nnz_local == 0 || col_idx_host != nullptr) && b_bounds != nullptr,
                 "null array");
  HPSPMM_REQUIRE(ctx, exchange == HPSPMM_EXCHANGE_NEEDED_ROWS || exchange == HPSPMM_EXCHANGE_ALL_ROWS ||
                          exchange == HPSPMM_EXCHANGE_NEEDED_ROWS_NCCL,
                 "unknown exchange mode");
  if (N > 2147483646ll || nnz_local > 2147483647ll - 4096) return HPSPMM_ERR_UNSUPPORTED;
  const int world = comm->world, rank = comm->rank;
  HPSPMM_REQUIRE(ctx, b_bounds[0] == 0 && b_bounds[world] == N, "b_bounds must run from 0 to N");
  for (int s = 0; s < world; ++s) HPSPMM_REQUIRE(ctx, b_bounds[s] <= b_bounds[s + 1], "b_bounds must ascend");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t us = (cudaStream_t)stream;

  hpspmm_shard_plan* p = new (std::nothrow) hpspmm_shard_plan();
  if (!p) return HPSPMM_ERR_OOM;
  p->device = ctx->device;
  p->world = world;
  p->rank = rank;
  p->comm = comm;
  p->exchange = exchange;
  p->M_local = M_local;
  p->N = N;
  p->nnz_local = nnz_local;
  p->max_K = max_K;
  p->rows_own = b_bounds[rank + 1] - b_bounds[rank];
  p->d_row_ptr = p->d_col = p->d_send_rows = nullptr;
  p->d_token = nullptr;
  p->push = exchange == HPSPMM_EXCHANGE_NEEDED_ROWS && world <= kMaxPushWorld;
  p->comm_stream = nullptr;
  // Grid of the push kernel (64-thread blocks, the product kernels' block size, so that a push block fits the slot
  // a finished product block leaves).  Measured on two B200s (315 MB per step in the busier direction) with the
  // same number of threads in 256-thread blocks: 2 / 4 / 8 / 16 such blocks per SM move the rows in 0.72 / 0.61 /
  // 0.54 / 0.51 ms -- remote stores need many threads in flight to fill the link.  A smaller grid overlaps better
  // with the product beside it (0.2 ms hidden at 2 blocks per SM against 0.07 at 16) but the step comes out the
  // same, so the grid that finishes the exchange soonest is kept.  Packing locally and letting the copy engines
  // carry the blocks (cudaMemcpyAsync to the peer mapping) was slower: 0.87 ms for the same rows, and a longer
  // step.  So was a variant that gathers tiles of rows into shared memory (cp.async) and hands each tile to the
  // bulk-copy engine as one 16 KB store to the peer mapping (cp.async.bulk shared -> global), meant to fill the
  // link from two small blocks per SM: 0.88 ms at two blocks per SM, 0.68 ms at four -- a bulk store to a peer
  // completes too slowly for so few of them in flight.  HPSPMM_PUSH_BLOCKS overrides (tuning aid).
  p->push_blocks = (int64_t)ctx->sm_count * 64;
  if (const char* env = getenv("HPSPMM_PUSH_BLOCKS")) {
    const long v = atol(env);
    if (v > 0) p->push_blocks = v;
  }
  p->device_bytes = 0;
  memset(p->slots, 0, sizeof(p->slots));

  // which rows of B the shard names, per owner, and the shard's columns in that compact numbering
  std::vector<int32_t> col_compact((size_t)std::max<int64_t>(nnz_local, 1));
  std::vector<int32_t> need_rows;
  std::vector<int64_t> need_off((size_t)world + 1);
  int st = HPSPMM_OK;
  const bool needed_only = exchange != HPSPMM_EXCHANGE_ALL_ROWS;
  if (needed_only) {
    need_rows.resize((size_t)std::min<int64_t>(N, std::max<int64_t>(nnz_local, 1)));
    st = hpspmm_shard_needed_rows(nnz_local, col_idx_host, N, world, b_bounds, col_compact.data(), need_rows.data(),
                                  need_off.data(), &p->n_needed);
  } else {
    for (int s = 0; s <= world; ++s) need_off[s] = b_bounds[s];
    p->n_needed = N;
    if (nnz_local > 0) memcpy(col_compact.data(), col_idx_host, (size_t)nnz_local * 4);
  }
  p->recv_off.assign(need_off.begin(), need_off.end());

  // counts: every rank learns how many rows every other rank wants from it
  std::vector<int32_t> want((size_t)world), all_want((size_t)world * world);
  for (int s = 0; s < world; ++s) want[s] = (int32_t)(need_off[s + 1] - need_off[s]);
  cudaError_t e = cudaSuccess;
  int32_t* d_cnt = nullptr;
  const nccl_api* api = comm->api;
#define PLAN_FAIL(status)        \
  do {                           \
    if (d_cnt) cudaFree(d_cnt);  \
    hpspmm_shard_plan_destroy(ctx, p); \
    return (status);             \
  } while (0)
  if (st != HPSPMM_OK) PLAN_FAIL(st);
  {
    // highest priority: the exchange is short on SM work and long on link time, so its blocks should get the
    // next free SM slots ahead of the product that runs beside it
    int lo_prio = 0, hi_prio = 0;
    cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio);
    if (cudaStreamCreateWithPriority(&p->comm_stream, cudaStreamNonBlocking, hi_prio) != cudaSuccess)
      PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "comm stream", cudaGetLastError()));
  }
  if (world > 1) {
    e = hpspmm_device_malloc((void**)&d_cnt, (size_t)(world + 1) * world * 4);
    if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_OOM, "plan cudaMalloc", e));
    e = cudaMemcpyAsync(d_cnt, want.data(), (size_t)world * 4, cudaMemcpyHostToDevice, us);
    if (e == cudaSuccess) {
      const int rc = api->AllGather(d_cnt, d_cnt + world, (size_t)world, kNcclInt32, comm->comm, us);
      if (rc != 0) PLAN_FAIL(nccl_fail(ctx, api, "ncclAllGather(counts)", rc));
      e = cudaMemcpyAsync(all_want.data(), d_cnt + world, (size_t)world * world * 4, cudaMemcpyDeviceToHost, us);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(us);
    if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "count exchange", e));
  } else {
    all_want[0] = want[0];
  }
  p->send_cnt.assign((size_t)world, 0);
  for (int d = 0; d < world; ++d) p->send_cnt[d] = all_want[(size_t)d * world + rank];
  p->send_off.assign((size_t)world + 1, 0);
  {
    std::vector<int64_t> by_slot((size_t)world, 0);
    for (int d = 0; d < world; ++d) by_slot[send_slot_of(d, rank, world)] = p->send_cnt[d];
    for (int i = 0; i < world; ++i) p->send_off[i + 1] = p->send_off[i] + by_slot[i];
  }
  p->send_remote = p->send_off[world - 1];
  const int64_t send_total = p->send_off[world];
  // where this rank's block starts in rank d's dense operand: d wants all_want[d][s] rows from every s < rank first
  p->dst_first_row.assign((size_t)world, 0);
  for (int d = 0; d < world; ++d)
    for (int s2 = 0; s2 < rank; ++s2) p->dst_first_row[d] += all_want[(size_t)d * world + s2];
  for (int d = 0; d < world; ++d)
    if (p->send_cnt[d] > p->rows_own) {
      snprintf(ctx->err, sizeof(ctx->err), "rank %d asks for more rows than this rank owns", d);
      PLAN_FAIL(HPSPMM_ERR_INVALID);
    }

  // device copies: row_ptr, renumbered columns, the rows to send
  const size_t b_rp = align_up((size_t)(M_local + 1) * 4, 256);
  const size_t b_col = align_up((size_t)std::max<int64_t>(nnz_local, 1) * 4, 256);
  const size_t b_send = align_up((size_t)std::max<int64_t>(send_total, 1) * 4, 256);
  const size_t b_need = align_up((size_t)std::max<int64_t>(p->n_needed, 1) * 4, 256);
  char* base = nullptr;
  e = hpspmm_device_malloc((void**)&base, b_rp + b_col + b_send + b_need + 256);
  if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_OOM, "plan cudaMalloc", e));
  p->device_bytes += b_rp + b_col + b_send + b_need;
  p->d_row_ptr = (int32_t*)base;
  p->d_col = (int32_t*)(base + b_rp);
  p->d_send_rows = (int32_t*)(base + b_rp + b_col);
  int32_t* d_need = (int32_t*)(base + b_rp + b_col + b_send);   // only used while the lists are exchanged
  p->d_token = (int32_t*)(base + b_rp + b_col + b_send + b_need);
  if (cudaMemsetAsync(p->d_token, 0, 256, us) != cudaSuccess)
    PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "plan memset", cudaGetLastError()));
  e = cudaMemcpyAsync(p->d_row_ptr, row_ptr_host, (size_t)(M_local + 1) * 4, cudaMemcpyHostToDevice, us);
  if (e == cudaSuccess && nnz_local > 0)
    e = cudaMemcpyAsync(p->d_col, col_compact.data(), (size_t)nnz_local * 4, cudaMemcpyHostToDevice, us);
  if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "plan upload", e));

  if (needed_only) {
    // every owner receives the global ids of the rows wanted from it and makes them local
    if (p->n_needed > 0)
      e = cudaMemcpyAsync(d_need, need_rows.data(), (size_t)p->n_needed * 4, cudaMemcpyHostToDevice, us);
    if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "plan upload", e));
    const int self = send_slot_of(rank, rank, world);
    if (p->send_cnt[rank] > 0) {
      e = cudaMemcpyAsync(p->d_send_rows + p->send_off[self], d_need + need_off[rank], (size_t)p->send_cnt[rank] * 4,
                          cudaMemcpyDeviceToDevice, us);
      if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "plan copy", e));
    }
    if (world > 1) {
      int rc = api->GroupStart();
      for (int d = 0; d < world && rc == 0; ++d) {
        if (d == rank) continue;
        if (want[d] > 0) rc = api->Send(d_need + need_off[d], (size_t)want[d], kNcclInt32, d, comm->comm, us);
        if (rc == 0 && p->send_cnt[d] > 0)
          rc = api->Recv(p->d_send_rows + p->send_off[send_slot_of(d, rank, world)], (size_t)p->send_cnt[d], kNcclInt32,
                         d, comm->comm, us);
      }
      const int rc2 = api->GroupEnd();
      if (rc != 0 || rc2 != 0) PLAN_FAIL(nccl_fail(ctx, api, "row list exchange", rc != 0 ? rc : rc2));
    }
    if (send_total > 0) {
      rebase_rows_kernel<<<(unsigned)((send_total + 255) / 256), 256, 0, us>>>(p->d_send_rows, send_total,
                                                                             (int)b_bounds[rank]);
      ctx->launches++;
    }
  }
  e = cudaStreamSynchronize(us);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "shard plan build", e));
  if (needed_only && send_total > 0) {
    // a malformed request (a row outside this rank's block) must not turn into a wild gather
    std::vector<int32_t> chk((size_t)send_total);
    e = cudaMemcpy(chk.data(), p->d_send_rows, (size_t)send_total * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) PLAN_FAIL(hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "plan check", e));
    for (int64_t i = 0; i < send_total; ++i)
      if (chk[i] < 0 || chk[i] >= p->rows_own) {
        snprintf(ctx->err, sizeof(ctx->err), "a rank asked for a row this rank does not own");
        PLAN_FAIL(HPSPMM_ERR_INVALID);
      }
  }
  if (d_cnt) cudaFree(d_cnt);
#undef PLAN_FAIL
  *out = p;
  return HPSPMM_OK;
}

int hpspmm_shard_plan_destroy(hpspmm_ctx* ctx, hpspmm_shard_plan* p) {
  if (!p) return HPSPMM_OK;
  hpspmm_device_guard guard(p->device);
  cudaDeviceSynchronize();
  // unmap everything first, meet once, then free (see meet_all_ranks)
  bool any = false;
  for (int i = 0; i < kSlots; ++i) any = close_peer_mappings(p->slots[i]) || any;
  if (any) meet_all_ranks(p);
  for (int i = 0; i < kSlots; ++i) {
    hpspmm_shard_slot& s = p->slots[i];
    release_slot_buffers(ctx, p, s);
    if (s.ev_in) cudaEventDestroy(s.ev_in);
    if (s.ev_landed) cudaEventDestroy(s.ev_landed);
    if (s.ev_read) cudaEventDestroy(s.ev_read);
  }
  if (p->d_row_ptr) cudaFree(p->d_row_ptr);
  if (p->comm_stream) cudaStreamDestroy(p->comm_stream);
  delete p;
  return HPSPMM_OK;
}

int hpspmm_shard_plan_info(const hpspmm_shard_plan* p, int64_t* rows_local, int64_t* rows_received,
                           int64_t* rows_sent, int64_t* device_bytes) {
  if (!p) return HPSPMM_ERR_INVALID;
  if (rows_local) *rows_local = p->n_needed;
  if (rows_received) *rows_received = p->n_needed - (p->recv_off[p->rank + 1] - p->recv_off[p->rank]);
  if (rows_sent) *rows_sent = p->send_remote;
  if (device_bytes) *device_bytes = (int64_t)p->device_bytes;
  return HPSPMM_OK;
}

int hpspmm_sharded_exchange_begin(hpspmm_ctx* ctx, hpspmm_shard_plan* p, int32_t slot, int64_t K, const float* B_own,
                                  hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_sharded_exchange_begin");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && p != nullptr, "null context or plan");
  HPSPMM_REQUIRE(ctx, p->device == ctx->device, "plan built on another device");
  HPSPMM_REQUIRE(ctx, slot >= 0 && slot < kSlots, "slot out of range");
  HPSPMM_REQUIRE(ctx, K >= 1 && K <= p->max_K, "K outside the plan's range");
  HPSPMM_REQUIRE(ctx, p->rows_own == 0 || B_own != nullptr, "null B_own");
  HPSPMM_REQUIRE(ctx, (K & 3) != 0 || ((uintptr_t)B_own & 15u) == 0, "B_own must be 16-byte aligned");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t us = (cudaStream_t)stream, cs = p->comm_stream;
  int st = ensure_slot(ctx, p, slot, K, us);
  if (st != HPSPMM_OK) return st;
  hpspmm_shard_slot& s = p->slots[slot];
  const int world = p->world, rank = p->rank;
  HPSPMM_REQUIRE(ctx, !s.begun, "the slot was begun again before its product was enqueued");
  // the exchange starts once B_own is ready and the last product of this slot has read its buffer
  HPSPMM_CUDA_TRY(ctx, cudaEventRecord(s.ev_in, us));
  HPSPMM_CUDA_TRY(ctx, cudaStreamWaitEvent(cs, s.ev_in, 0));
  if (s.read_pending) HPSPMM_CUDA_TRY(ctx, cudaStreamWaitEvent(cs, s.ev_read, 0));
  s.read_pending = false;
  const int self = send_slot_of(rank, rank, world);
  if (p->push) {
    // one kernel stores every referenced row where it will be read: the other ranks' operands through their
    // peer mappings, this rank's own rows into its own operand
    s.phase ^= 1;
    const int b = s.phase;
    const int64_t total_rows = p->send_off[world];
    if (total_rows > 0) {
      push_targets t;
      memset(&t, 0, sizeof(t));
      t.n = world;
      for (int d = 0; d < world; ++d) {
        const int pos = send_slot_of(d, rank, world);
        t.base[pos] = d == rank ? s.B_local[b] : s.peer[b][d];
        t.first_row[pos] = p->dst_first_row[d];
        t.list_begin[pos] = p->send_off[pos];
      }
      t.list_begin[world] = total_rows;
      const bool vec = (K & 3) == 0;
      const int64_t row_elems = vec ? K / 4 : K;
      int64_t blocks = (total_rows * row_elems + kPushThreads - 1) / kPushThreads;
      const int64_t cap = p->push_blocks;
      if (blocks > cap) blocks = cap;
      if (vec)
        push_rows_kernel<4><<<(unsigned)blocks, kPushThreads, 0, cs>>>(B_own, p->d_send_rows, total_rows, row_elems, t);
      else
        push_rows_kernel<1><<<(unsigned)blocks, kPushThreads, 0, cs>>>(B_own, p->d_send_rows, total_rows, row_elems, t);
      ctx->launches++;
      HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
    }
    if (world > 1) {
      // completion signal: finished here = every rank's push kernel has ended
      const nccl_api* api = p->comm->api;
      HPSPMM_NCCL_TRY(ctx, api, api->AllReduce(p->d_token, p->d_token + 1, 1, kNcclInt32, kNcclSum, p->comm->comm, cs));
    }
    HPSPMM_CUDA_TRY(ctx, cudaEventRecord(s.ev_landed, cs));
    s.begun = true;
    return HPSPMM_OK;
  }
  float* Bl = s.B_local[0];
  float* own_dst = Bl + p->recv_off[rank] * K;
  if (p->exchange != HPSPMM_EXCHANGE_ALL_ROWS) {
    // rows for the others -> send buffer; own referenced rows -> straight into their place
    if (p->send_remote > 0) {
      st = hpspmm_gather_rows_f32(ctx, p->send_remote, K, B_own, p->d_send_rows, s.send_buf, (hpspmm_stream)cs);
      if (st != HPSPMM_OK) return st;
    }
    if (p->send_cnt[rank] > 0) {
      st = hpspmm_gather_rows_f32(ctx, p->send_cnt[rank], K, B_own, p->d_send_rows + p->send_off[self], own_dst,
                                  (hpspmm_stream)cs);
      if (st != HPSPMM_OK) return st;
    }
  } else if (p->rows_own > 0) {
    HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(own_dst, B_own, (size_t)p->rows_own * (size_t)K * 4, cudaMemcpyDeviceToDevice, cs));
  }
  if (world > 1) {
    const nccl_api* api = p->comm->api;
    int rc = api->GroupStart();
    for (int d = 0; d < world && rc == 0; ++d) {
      if (d == rank) continue;
      const int64_t n_recv = p->recv_off[d + 1] - p->recv_off[d];
      if (p->exchange != HPSPMM_EXCHANGE_ALL_ROWS) {
        if (p->send_cnt[d] > 0)
          rc = api->Send(s.send_buf + p->send_off[send_slot_of(d, rank, world)] * K, (size_t)(p->send_cnt[d] * K),
                         kNcclFloat32, d, p->comm->comm, cs);
      } else if (p->rows_own > 0) {
        rc = api->Send(B_own, (size_t)(p->rows_own * K), kNcclFloat32, d, p->comm->comm, cs);
      }
      if (rc == 0 && n_recv > 0)
        rc = api->Recv(Bl + p->recv_off[d] * K, (size_t)(n_recv * K), kNcclFloat32, d, p->comm->comm, cs);
    }
    const int rc2 = api->GroupEnd();
    if (rc != 0 || rc2 != 0) return nccl_fail(ctx, api, "row exchange", rc != 0 ? rc : rc2);
  }
  HPSPMM_CUDA_TRY(ctx, cudaEventRecord(s.ev_landed, cs));
  s.begun = true;
  return HPSPMM_OK;
}

int hpspmm_sharded_product(hpspmm_ctx* ctx, hpspmm_shard_plan* p, int32_t slot, int64_t K, const float* vals,
                           float* C_local, const hpspmm_opts* opts, hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_sharded_product");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && p != nullptr, "null context or plan");
  HPSPMM_REQUIRE(ctx, slot >= 0 && slot < kSlots, "slot out of range");
  hpspmm_shard_slot& s = p->slots[slot];
  HPSPMM_REQUIRE(ctx, s.plan != nullptr && K >= 1 && K <= s.K_cap, "no exchange of this width was begun on the slot");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t us = (cudaStream_t)stream;
  HPSPMM_CUDA_TRY(ctx, cudaStreamWaitEvent(us, s.ev_landed, 0));
  int st = hpspmm_spmm_csr_f32(ctx, s.plan, p->M_local, p->n_needed, K, p->nnz_local, p->d_row_ptr, p->d_col, vals,
                               s.B_local[p->push ? s.phase : 0], C_local, opts, stream);
  if (st != HPSPMM_OK) return st;
  HPSPMM_CUDA_TRY(ctx, cudaEventRecord(s.ev_read, us));
  s.read_pending = true;
  s.begun = false;
  return HPSPMM_OK;
}

int hpspmm_spmm_sharded_f32(hpspmm_ctx* ctx, hpspmm_shard_plan* plan, int64_t K, const float* vals, const float* B_own,
                            float* C_local, const hpspmm_opts* opts, hpspmm_stream stream) {
  int st = hpspmm_sharded_exchange_begin(ctx, plan, 0, K, B_own, stream);
  if (st != HPSPMM_OK) return st;
  return hpspmm_sharded_product(ctx, plan, 0, K, vals, C_local, opts, stream);
}

}  // extern "C"
