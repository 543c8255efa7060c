// Multi-GPU side of the quantize-and-execute path: one communicator per GPU (one process per GPU, or one host thread
// per GPU inside one process), NCCL for the three exchanges the path has.
//
//   whole-model quantization   tensors go to ranks whole (largest first); a tensor larger than the split threshold is cut
//                              into row blocks, and for a per-tensor scale the ranks combine their partial absmax with a
//                              MAX all-reduce of ONE float per split tensor.  Codes never leave their GPU.
//   W4A16 / FP8 GEMM           column-parallel: every rank owns N/world output columns of W with their scales / zero
//                              points, runs the tensor-core kernel on its own memory, then ncclAllGather brings the
//                              M x N/world bf16 blocks together in every rank's own memory.
//   GPTQ                       output rows are sharded, U is replicated; the Hessian may be accumulated token-parallel
//                              and summed with one all-reduce of K x K floats.
//
// The reference only stamps `castforge.all_gather` / `castforge.all_reduce` attributes on its graph
// (src/passes/distributed/spmd.rs:416-478) and evaluates them as the identity (src/codegen/eval.rs:1449-1455); there is
// no communication code to follow.  NCCL is opened at run time (dlopen of libnccl.so.2), so the library loads and every
// single-GPU entry point works on a machine without NCCL; only the calls below need it.
//
// Rejoining the column-parallel blocks.  Where the ranks are separate processes on one node, every rank keeps its GEMM
// output block in a buffer the others have mapped (CUDA IPC), and after one small all-reduce (the "every block is
// complete" barrier) a copy kernel of this library reads the peers' blocks over NVLink with plain 16-byte loads and
// writes them straight to their columns of the row-major result: one pass over the product instead of NCCL's all-gather
// into a staging area plus an interleave pass.  No TMA, no multicast, no library kernel ever sees a peer pointer; if the
// mapping cannot be set up (ranks in one process, no peer access) the NCCL path is what runs.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "common.cuh"

struct cfb200_comm {
  ncclComm_t nccl = nullptr;
  int world = 1, rank = 0, device = 0;
  // a side stream for small collectives that should not sit in the caller's stream between two kernels
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  // exchange buffer for the column-parallel products: two halves used by alternate calls, mapped by every peer
  static constexpr int kMaxPeers = 16;
  int xstate = 0;                 // 0 = not tried yet, 1 = mapped everywhere, -1 = not available (NCCL all-gather instead)
  void* xlocal = nullptr;         // this rank's buffer (cudaMalloc), 2 * xhalf bytes
  size_t xhalf = 0;
  void* xpeer[kMaxPeers] = {};    // xpeer[r] = rank r's buffer as mapped here (xpeer[rank] == xlocal)
  std::vector<void*> xretired;    // outgrown buffers and their mappings, released with the communicator
  std::vector<void*> xretired_maps;
  int32_t* xtick = nullptr;       // one device word for the barrier all-reduce
  unsigned xcalls = 0;
};

namespace cfb {
namespace {

struct NcclApi {
  void* handle = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclCommInitAll) CommInitAll = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  decltype(&ncclAllReduce) AllReduce = nullptr;
  decltype(&ncclGroupStart) GroupStart = nullptr;
  decltype(&ncclGroupEnd) GroupEnd = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclGetVersion) GetVersion = nullptr;
};

NcclApi g_nccl;
std::mutex g_nccl_mutex;

// Opens NCCL once.  A process that already carries libnccl.so.2 (PyTorch loads its own copy) gets that copy back.
int32_t nccl_api(const NcclApi** out) {
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (!g_nccl.handle) {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return set_error(CFB200_ERR_UNSUPPORTED, "NCCL is not available: %s", dlerror());
    NcclApi a;
    a.handle = h;
#define CFB_SYM(field, name)                                                                         \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(h, name));                                     \
  if (!a.field) return set_error(CFB200_ERR_UNSUPPORTED, "NCCL symbol %s is missing", name)
    CFB_SYM(GetUniqueId, "ncclGetUniqueId");
    CFB_SYM(CommInitRank, "ncclCommInitRank");
    CFB_SYM(CommInitAll, "ncclCommInitAll");
    CFB_SYM(CommDestroy, "ncclCommDestroy");
    CFB_SYM(AllGather, "ncclAllGather");
    CFB_SYM(AllReduce, "ncclAllReduce");
    CFB_SYM(GroupStart, "ncclGroupStart");
    CFB_SYM(GroupEnd, "ncclGroupEnd");
    CFB_SYM(GetErrorString, "ncclGetErrorString");
    CFB_SYM(GetVersion, "ncclGetVersion");
#undef CFB_SYM
    g_nccl = a;
  }
  *out = &g_nccl;
  return CFB200_OK;
}

#define CFB_NCCL(api, call)                                                                            \
  do {                                                                                                 \
    ncclResult_t r__ = (call);                                                                         \
    if (r__ != ncclSuccess) return set_error(CFB200_ERR_CUDA, "%s failed: %s", #call, (api)->GetErrorString(r__)); \
  } while (0)

// gathered [world][M][Nl] (what ncclAllGather leaves) -> row-major [M][world * Nl], 16 bytes per thread
__global__ void interleave_blocks_kernel(const uint4* __restrict__ gathered, uint4* __restrict__ out, size_t M, size_t vec_per_row_local,
                                         int world) {
  const size_t total = (size_t)world * M * vec_per_row_local;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t v = i % vec_per_row_local, rm = i / vec_per_row_local;
    const size_t m = rm % M, r = rm / M;
    out[(m * world + r) * vec_per_row_local + v] = gathered[i];
  }
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// ---- peer-mapped exchange buffer ----------------------------------------------------------------------------------------
struct XInfo {
  cudaIpcMemHandle_t handle;
  int32_t pid, ok;
};

// Collective over the communicator: makes sure every rank owns an exchange buffer of 2 * half_bytes that every other rank
// has mapped.  Leaves comm->xstate at 1 (mapped) or -1 (fall back to NCCL) -- the same value on every rank.
int32_t ensure_exchange(cfb200_comm* comm, size_t half_bytes, cudaStream_t st) {
  if (comm->xstate < 0) return CFB200_OK;
  if (comm->xstate == 1 && comm->xhalf >= half_bytes) return CFB200_OK;
  const NcclApi* api;
  int32_t rc = nccl_api(&api);
  if (rc) return rc;
  const int W = comm->world;
  if (W > cfb200_comm::kMaxPeers) { comm->xstate = -1; return CFB200_OK; }
  // the buffers in use go on the retired list (a peer may still be reading them); they are released with the communicator
  if (comm->xlocal) {
    comm->xretired.push_back(comm->xlocal);
    for (int r = 0; r < W; ++r)
      if (r != comm->rank && comm->xpeer[r]) comm->xretired_maps.push_back(comm->xpeer[r]);
    comm->xlocal = nullptr;
    for (int r = 0; r < W; ++r) comm->xpeer[r] = nullptr;
  }
  const size_t half = align256(half_bytes + half_bytes / 4);  // some headroom: growing is a collective with two host round trips
  XInfo mine;
  memset(&mine, 0, sizeof mine);
  mine.pid = (int32_t)getpid();
  mine.ok = 1;
  void* buf = nullptr;
  if (cudaMalloc(&buf, 2 * half) != cudaSuccess) { cudaGetLastError(); buf = nullptr; mine.ok = 0; }
  struct PendingBuffer {  // the new exchange buffer belongs to this function until the ranks have agreed to use it
    void* p = nullptr;
    ~PendingBuffer() { if (p) cudaFree(p); }
  } pending;
  pending.p = buf;
  if (mine.ok && cudaIpcGetMemHandle(&mine.handle, buf) != cudaSuccess) { cudaGetLastError(); mine.ok = 0; }
  if (!comm->xtick) {
    CFB_CUDA(cudaMalloc(reinterpret_cast<void**>(&comm->xtick), 256));
    CFB_CUDA(cudaMemsetAsync(comm->xtick, 0, 256, st));
  }
  // every rank's record to every rank (through device memory: NCCL moves device buffers)
  struct DevScratch {  // released on every way out of this function
    XInfo* p = nullptr;
    ~DevScratch() { if (p) cudaFree(p); }
  } dev_all;
  CFB_CUDA(cudaMalloc(reinterpret_cast<void**>(&dev_all.p), sizeof(XInfo) * W));
  CFB_CUDA(cudaMemcpyAsync(dev_all.p + comm->rank, &mine, sizeof mine, cudaMemcpyHostToDevice, st));
  CFB_NCCL(api, api->AllGather(dev_all.p + comm->rank, dev_all.p, sizeof(XInfo), ncclInt8, comm->nccl, st));
  std::vector<XInfo> all(W);
  CFB_CUDA(cudaMemcpyAsync(all.data(), dev_all.p, sizeof(XInfo) * W, cudaMemcpyDeviceToHost, st));
  CFB_CUDA(cudaStreamSynchronize(st));
  int good = 1;
  for (int r = 0; r < W; ++r) {
    if (!all[r].ok) good = 0;
    if (r != comm->rank && all[r].pid == mine.pid) good = 0;  // ranks inside one process: an IPC handle cannot be opened there
  }
  void* maps[cfb200_comm::kMaxPeers] = {};
  if (good) {
    for (int r = 0; r < W && good; ++r) {
      if (r == comm->rank) { maps[r] = buf; continue; }
      if (cudaIpcOpenMemHandle(&maps[r], all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        maps[r] = nullptr;
        good = 0;
      }
    }
  }
  auto close_maps = [&]() {
    for (int r = 0; r < W; ++r)
      if (r != comm->rank && maps[r]) { cudaIpcCloseMemHandle(maps[r]); maps[r] = nullptr; }
  };
  // agree: one rank that could not map means nobody uses the mapping
  int32_t vote = good;
  int32_t* dev_vote = reinterpret_cast<int32_t*>(dev_all.p);
  bool agreed = cudaMemcpyAsync(dev_vote, &vote, sizeof vote, cudaMemcpyHostToDevice, st) == cudaSuccess &&
                api->AllReduce(dev_vote, dev_vote, 1, ncclInt32, ncclMin, comm->nccl, st) == ncclSuccess &&
                cudaMemcpyAsync(&vote, dev_vote, sizeof vote, cudaMemcpyDeviceToHost, st) == cudaSuccess &&
                cudaStreamSynchronize(st) == cudaSuccess;
  if (!agreed) {
    close_maps();
    comm->xstate = -1;
    return set_error(CFB200_ERR_CUDA, "the ranks could not agree on the exchange buffers (CUDA or NCCL error)");
  }
  if (vote == 1) {
    comm->xlocal = buf;
    pending.p = nullptr;  // kept
    comm->xhalf = half;
    for (int r = 0; r < W; ++r) comm->xpeer[r] = maps[r];
    comm->xstate = 1;
  } else {
    close_maps();
    comm->xstate = -1;  // (the buffer goes with `pending`)
  }
  return CFB200_OK;
}

struct PullArgs {
  const uint4* src[cfb200_comm::kMaxPeers];
};
// every rank's [M, Nl] block (in that rank's exchange buffer, read through its mapping here) -> this rank's result:
// row-major [M][world * Nl] (layout 0) or [world][M][Nl] (layout 1).  16 bytes per load, four loads in flight per thread;
// consecutive threads read consecutive vectors of one block row, consecutive rows come from different ranks.
#ifndef CFB_PULL_INFLIGHT
#define CFB_PULL_INFLIGHT 4
#endif
constexpr int kPullInFlight = CFB_PULL_INFLIGHT;  // 16-byte loads a thread has in flight
__global__ void __launch_bounds__(256) pull_blocks_kernel(PullArgs a, uint4* __restrict__ out, size_t M, size_t vpr, int world, int layout) {
  const size_t total = (size_t)world * M * vpr;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += kPullInFlight * step) {
    uint4 v[kPullInFlight];
    size_t dst[kPullInFlight];
#pragma unroll
    for (int u = 0; u < kPullInFlight; ++u) {
      const size_t i = i0 + u * step;
      if (i < total) {
        const size_t vv = i % vpr, mr = i / vpr;
        const size_t r = mr % world, m = mr / world;
        v[u] = a.src[r][m * vpr + vv];
        dst[u] = layout == 0 ? (m * world + r) * vpr + vv : (r * M + m) * vpr + vv;
      }
    }
#pragma unroll
    for (int u = 0; u < kPullInFlight; ++u)
      if (i0 + u * step < total) out[dst[u]] = v[u];
  }
}

// Small products stay with NCCL's all-gather: the barrier all-reduce in front of the peer loads costs about as much as
// the whole all-gather of a few hundred KB per rank (decode shapes).  "colpar_p2p": 0 = never, 1 = from 8 MB of product,
// n > 1 = from n MB, negative = always.
bool use_peer_loads(size_t block_bytes, int world) {
  const long long knob = tunable(kTuneColparP2P);
  if (knob == 0) return false;
  if (knob < 0) return true;
  return block_bytes * (size_t)world >= ((size_t)(knob == 1 ? 8 : knob) << 20);
}

// The block this rank is about to compute goes here (nullptr: no mapped exchange buffer, use the caller's workspace).
void* exchange_slot(cfb200_comm* comm) {
  if (comm->xstate != 1) return nullptr;
  return static_cast<char*>(comm->xlocal) + (size_t)(comm->xcalls & 1u) * comm->xhalf;
}

// After the local block has been written to exchange_slot(): barrier, then pull every block into C.
int32_t pull_columns(cfb200_comm* comm, size_t M, size_t Nl, size_t elem_bytes, void* C, int32_t layout, cudaStream_t st) {
  const NcclApi* api;
  int32_t rc = nccl_api(&api);
  if (rc) return rc;
  // every rank's block is complete (and everybody has finished reading the other half, which the next call overwrites)
  CFB_NCCL(api, api->AllReduce(comm->xtick, comm->xtick, 1, ncclInt32, ncclSum, comm->nccl, st));
  PullArgs a;
  const size_t off = (size_t)(comm->xcalls & 1u) * comm->xhalf;
  for (int r = 0; r < comm->world; ++r) a.src[r] = reinterpret_cast<const uint4*>(static_cast<const char*>(comm->xpeer[r]) + off);
  const size_t vpr = Nl * elem_bytes / 16;
  const size_t total = (size_t)comm->world * M * vpr;
  size_t blocks = (total / kPullInFlight + 255) / 256 + 1, cap = (size_t)sm_count() * 8;
  pull_blocks_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(a, reinterpret_cast<uint4*>(C), M, vpr, comm->world, layout);
  CFB_LAUNCH_CHECK();
  ++comm->xcalls;
  return CFB200_OK;
}

// local [M, Nl] block (elem_bytes per element) -> every rank's C [M, world * Nl] (layout 0) or [world][M][Nl] (layout 1)
int32_t gather_columns(cfb200_comm* comm, const void* part, size_t M, size_t Nl, size_t elem_bytes, void* C, int32_t layout,
                       void* gather_ws, cudaStream_t st) {
  const NcclApi* api;
  int32_t rc = nccl_api(&api);
  if (rc) return rc;
  const size_t block_bytes = M * Nl * elem_bytes;
  const bool direct = layout == 1 || M == 1 || comm->world == 1;  // the gathered order already is the wanted order
  void* dst = direct ? C : gather_ws;
  CFB_NCCL(api, api->AllGather(part, dst, block_bytes, ncclInt8, comm->nccl, st));
  if (!direct) {
    const size_t vpr = Nl * elem_bytes / 16;
    const size_t total = (size_t)comm->world * M * vpr;
    size_t blocks = (total + 255) / 256, cap = (size_t)sm_count() * 8;
    interleave_blocks_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(reinterpret_cast<const uint4*>(gather_ws),
                                                                                    reinterpret_cast<uint4*>(C), M, vpr, comm->world);
    CFB_LAUNCH_CHECK();
  }
  return CFB200_OK;
}

}  // namespace
}  // namespace cfb

using namespace cfb;

// ---- communicators --------------------------------------------------------------------------------------------------
extern "C" int32_t cfb200_comm_unique_id(void* id_out_128_host) {
  CFB_CHECK_ARG(id_out_128_host != nullptr, "NULL argument");
  static_assert(sizeof(ncclUniqueId) == 128, "the id travels as 128 opaque bytes");
  const NcclApi* api;
  int32_t rc = nccl_api(&api);
  if (rc) return rc;
  ncclUniqueId id;
  CFB_NCCL(api, api->GetUniqueId(&id));
  memcpy(id_out_128_host, &id, sizeof id);
  return CFB200_OK;
}

extern "C" int32_t cfb200_comm_init(const void* id_128_host, int32_t world, int32_t rank, cfb200_comm** comm_out) {
  CFB_CHECK_ARG(id_128_host && comm_out, "NULL argument");
  CFB_CHECK_ARG(world >= 1 && rank >= 0 && rank < world, "bad world / rank (%d, %d)", world, rank);
  *comm_out = nullptr;
  const NcclApi* api;
  int32_t rc = nccl_api(&api);
  if (rc) return rc;
  ncclUniqueId id;
  memcpy(&id, id_128_host, sizeof id);
  cfb200_comm* c = new cfb200_comm;
  c->world = world;
  c->rank = rank;
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return set_error(CFB200_ERR_CUDA, "cudaGetDevice failed"); }
  ncclResult_t r = api->CommInitRank(&c->nccl, world, id, rank);
  if (r != ncclSuccess) { delete c; return set_error(CFB200_ERR_CUDA, "ncclCommInitRank failed: %s", api->GetErrorString(r)); }
  *comm_out = c;
  return CFB200_OK;
}

extern "C" int32_t cfb200_comm_init_local(int32_t ndev, const int32_t* devices, cfb200_comm** comms_out) {
  CFB_CHECK_ARG(ndev >= 1 && ndev <= 64 && comms_out, "bad arguments");
  const NcclApi* api;
  int32_t rc = nccl_api(&api);
  if (rc) return rc;
  std::vector<int> devs(ndev);
  for (int i = 0; i < ndev; ++i) devs[i] = devices ? devices[i] : i;
  std::vector<ncclComm_t> raw(ndev, nullptr);
  CFB_NCCL(api, api->CommInitAll(raw.data(), ndev, devs.data()));
  for (int i = 0; i < ndev; ++i) {
    cfb200_comm* c = new cfb200_comm;
    c->nccl = raw[i];
    c->world = ndev;
    c->rank = i;
    c->device = devs[i];
    comms_out[i] = c;
  }
  return CFB200_OK;
}

extern "C" int32_t cfb200_comm_world(const cfb200_comm* comm) { return comm ? comm->world : 0; }
extern "C" int32_t cfb200_comm_rank(const cfb200_comm* comm) { return comm ? comm->rank : -1; }

extern "C" void cfb200_comm_free(cfb200_comm* comm) {
  if (!comm) return;
  const NcclApi* api;
  if (comm->xlocal || !comm->xretired.empty()) {
    // This rank's mappings of the peers' buffers are closed.  Its OWN exchange buffers stay allocated until the process
    // ends: a buffer may only be freed once no peer has it mapped, and learning that would take a collective here -- which
    // would hang the ranks that are shutting down cleanly whenever another rank has failed.  (One buffer pair per
    // communicator that ever ran a large column-parallel product.)
    int dev = 0;
    cudaGetDevice(&dev);
    cudaSetDevice(comm->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < comm->world && r < cfb200_comm::kMaxPeers; ++r)
      if (r != comm->rank && comm->xpeer[r]) cudaIpcCloseMemHandle(comm->xpeer[r]);
    for (void* m : comm->xretired_maps) cudaIpcCloseMemHandle(m);
    cudaSetDevice(dev);
  }
  if (comm->xtick) cudaFree(comm->xtick);
  if (comm->nccl && nccl_api(&api) == CFB200_OK) api->CommDestroy(comm->nccl);
  if (comm->ev_fork) cudaEventDestroy(comm->ev_fork);
  if (comm->ev_join) cudaEventDestroy(comm->ev_join);
  if (comm->side) cudaStreamDestroy(comm->side);
  delete comm;
}

extern "C" int32_t cfb200_nccl_version(int32_t* version_out) {
  CFB_CHECK_ARG(version_out != nullptr, "NULL argument");
  const NcclApi* api;
  int32_t rc = nccl_api(&api);
  if (rc) return rc;
  int v = 0;
  CFB_NCCL(api, api->GetVersion(&v));
  *version_out = v;
  return CFB200_OK;
}

// ---- placement (pure host arithmetic, identical on every rank: nothing is exchanged) -------------------------------------
extern "C" int32_t cfb200_shard_assign(int32_t count, const size_t* nbytes, int32_t world, size_t split_min_bytes, int32_t* owner) {
  CFB_CHECK_ARG(count >= 0 && world >= 1 && (count == 0 || (nbytes && owner)), "bad arguments");
  std::vector<int> order;
  std::vector<unsigned long long> load(world, 0);
  for (int i = 0; i < count; ++i) {
    if (world > 1 && split_min_bytes > 0 && nbytes[i] >= split_min_bytes) {
      owner[i] = -1;  // cut into row blocks: every rank gets 1/world of it
      for (int r = 0; r < world; ++r) load[r] += nbytes[i] / world;
    } else order.push_back(i);
  }
  // largest first onto the least-loaded rank; equal sizes keep store order, ties go to the lowest rank
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return nbytes[a] > nbytes[b]; });
  for (int i : order) {
    int best = 0;
    for (int r = 1; r < world; ++r)
      if (load[r] < load[best]) best = r;
    owner[i] = best;
    load[best] += nbytes[i];
  }
  return CFB200_OK;
}

extern "C" int32_t cfb200_shard_row_range(size_t rows, int32_t world, int32_t rank, size_t align, size_t* row_begin, size_t* row_end) {
  CFB_CHECK_ARG(world >= 1 && rank >= 0 && rank < world && align >= 1 && row_begin && row_end, "bad arguments");
  const size_t units = (rows + align - 1) / align, base = units / world, extra = units % world;
  const size_t lo = (size_t)rank * base + ((size_t)rank < extra ? (size_t)rank : extra);
  const size_t hi = lo + base + ((size_t)rank < extra ? 1 : 0);
  *row_begin = lo * align < rows ? lo * align : rows;
  *row_end = hi * align < rows ? hi * align : rows;
  return CFB200_OK;
}

// ---- A1 over a sharded store --------------------------------------------------------------------------------------------
extern "C" int32_t cfb200_quant_sym_tensors_sharded(cfb200_comm* comm, int32_t count, const void* const* srcs, int32_t src_dtype,
                                                    const size_t* ns, const int32_t* is_row_block, int32_t bits,
                                                    int8_t* const* codes, float* scale_absmax, void* stream) {
  CFB_CHECK_ARG(comm != nullptr, "NULL communicator");
  CFB_CHECK_ARG(count >= 0, "negative count");
  if (count == 0) return CFB200_OK;
  CFB_CHECK_ARG(srcs && ns && codes && scale_absmax, "NULL argument");
  cudaStream_t st = (cudaStream_t)stream;
  std::vector<int> w_idx, blocks;
  for (int i = 0; i < count; ++i) {
    if (is_row_block && is_row_block[i]) blocks.push_back(i);
    else w_idx.push_back(i);
  }
  int32_t rc = CFB200_OK;
  // 1. row blocks: partial absmax on this rank, then one MAX all-reduce of one float per split tensor.  Every rank
  //    passes the split tensors in the same order (an empty block takes part with absmax 0).
  for (int i : blocks) {
    if (ns[i]) rc = cfb200_absmax(srcs[i], src_dtype, ns[i], scale_absmax + 2 * i + 1, st);
    else rc = cudaMemsetAsync(scale_absmax + 2 * i, 0, 2 * sizeof(float), st) == cudaSuccess ? CFB200_OK : set_error(CFB200_ERR_CUDA, "cudaMemsetAsync failed");
    if (rc) return rc;
  }
  // The all-reduce runs on the communicator's side stream, forked from the caller's stream after the absmax kernels and
  // joined before the first apply kernel, so that its latency (tens of microseconds for a few floats) passes under the
  // list kernel of the whole tensors instead of between two kernels.
  const bool exchange = !blocks.empty() && comm->world > 1;
  if (exchange) {
    const NcclApi* api;
    rc = nccl_api(&api);
    if (rc) return rc;
    if (!comm->side) {
      CFB_CUDA(cudaStreamCreateWithFlags(&comm->side, cudaStreamNonBlocking));
      CFB_CUDA(cudaEventCreateWithFlags(&comm->ev_fork, cudaEventDisableTiming));
      CFB_CUDA(cudaEventCreateWithFlags(&comm->ev_join, cudaEventDisableTiming));
    }
    CFB_CUDA(cudaEventRecord(comm->ev_fork, st));
    CFB_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_fork, 0));
    CFB_NCCL(api, api->GroupStart());
    for (int i : blocks) {
      ncclResult_t r = api->AllReduce(scale_absmax + 2 * i + 1, scale_absmax + 2 * i + 1, 1, ncclFloat32, ncclMax, comm->nccl, comm->side);
      if (r != ncclSuccess) { api->GroupEnd(); return set_error(CFB200_ERR_CUDA, "ncclAllReduce failed: %s", api->GetErrorString(r)); }
    }
    CFB_NCCL(api, api->GroupEnd());
    CFB_CUDA(cudaEventRecord(comm->ev_join, comm->side));
  }
  // 2. whole tensors: the list kernel on every maximal run of consecutive whole tensors (results land in place);
  //    it runs while the all-reduce above is still in flight on the same stream order
  for (size_t k = 0; k < w_idx.size();) {
    size_t e = k + 1;
    while (e < w_idx.size() && w_idx[e] == w_idx[e - 1] + 1) ++e;
    const int first = w_idx[k];
    rc = cfb200_quant_sym_tensors((int32_t)(e - k), srcs + first, src_dtype, ns + first, bits, codes + first,
                                  scale_absmax + 2 * first, 0, nullptr, stream);
    if (rc) return rc;
    k = e;
  }
  // 3. row blocks: codes from the global absmax
  if (exchange) CFB_CUDA(cudaStreamWaitEvent(st, comm->ev_join, 0));
  for (int i : blocks) {
    rc = cfb200_quant_sym_apply(srcs[i], src_dtype, ns[i], bits, scale_absmax + 2 * i + 1, codes[i], scale_absmax + 2 * i, stream);
    if (rc) return rc;
  }
  return CFB200_OK;
}

// ---- column-parallel GEMMs ------------------------------------------------------------------------------------------------
extern "C" size_t cfb200_gemm_colpar_workspace_bytes(size_t M, size_t N_local, size_t K, int32_t world, int32_t w4) {
  const size_t out_bytes = align256(M * N_local * 2);
  size_t need = out_bytes;                                     // this rank's [M, N_local] bf16 block
  if (world > 1 && M > 1) need += align256(out_bytes * world);  // the gathered blocks before they are interleaved
  if (w4 && M > 16) need += align256(cfb200_gemm_w4a16_workspace_bytes(M, N_local, K));
  return need;
}

extern "C" int32_t cfb200_gemm_w4a16_colpar(cfb200_comm* comm, const void* A, const uint8_t* w_codes, const uint16_t* w_scales,
                                            const uint8_t* w_zps, size_t M, size_t N_local, size_t K, size_t group, void* C,
                                            int32_t layout, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                                            void* stream) {
  CFB_CHECK_ARG(comm != nullptr, "NULL communicator");
  CFB_CHECK_ARG(layout == 0 || layout == 1, "layout must be 0 (row-major [M, N]) or 1 ([world][M][N_local])");
  CFB_CHECK_ARG(N_local % 8 == 0, "N_local must be a multiple of 8 (got %zu)", N_local);
  CFB_CHECK_ALIGNED(workspace, 256);
  CFB_CHECK_ALIGNED(C, 16);
  const size_t need = cfb200_gemm_colpar_workspace_bytes(M, N_local, K, comm->world, 1);
  if (!workspace || workspace_bytes < need) return set_error(CFB200_ERR_WORKSPACE, "gemm_w4a16_colpar needs %zu bytes of workspace", need);
  char* ws = reinterpret_cast<char*>(workspace);
  const size_t out_bytes = align256(M * N_local * 2);
  void* gathered = ws + out_bytes;
  const bool has_gather = comm->world > 1 && M > 1;
  void* inner = ws + out_bytes + (has_gather ? align256(out_bytes * comm->world) : 0);
  int32_t rc;
  const bool p2p = has_gather && use_peer_loads(out_bytes, comm->world);
  if (p2p) {
    rc = ensure_exchange(comm, out_bytes, (cudaStream_t)stream);
    if (rc) return rc;
  }
  void* slot = p2p ? exchange_slot(comm) : nullptr;
  void* part = slot ? slot : ws;
  if (M <= 16 && group == 128) rc = cfb200_gemv_w4a16(A, w_codes, w_scales, w_zps, M, N_local, K, group, part, 0, stream);
  else rc = cfb200_gemm_w4a16(A, w_codes, w_scales, w_zps, M, N_local, K, group, part, 0, inner,
                              cfb200_gemm_w4a16_workspace_bytes(M, N_local, K), error_flag, stream);
  if (rc) return rc;
  if (slot) return pull_columns(comm, M, N_local, 2, C, layout, (cudaStream_t)stream);
  return gather_columns(comm, part, M, N_local, 2, C, layout, gathered, (cudaStream_t)stream);
}

extern "C" int32_t cfb200_gemm_fp8_colpar(cfb200_comm* comm, const uint8_t* A, const float* a_scales, const uint8_t* W_local,
                                          float w_scale, size_t M, size_t N_local, size_t K, void* C, int32_t layout,
                                          void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream) {
  CFB_CHECK_ARG(comm != nullptr, "NULL communicator");
  CFB_CHECK_ARG(layout == 0 || layout == 1, "layout must be 0 (row-major [M, N]) or 1 ([world][M][N_local])");
  CFB_CHECK_ARG(N_local % 8 == 0, "N_local must be a multiple of 8 (got %zu)", N_local);
  CFB_CHECK_ALIGNED(workspace, 256);
  CFB_CHECK_ALIGNED(C, 16);
  const size_t need = cfb200_gemm_colpar_workspace_bytes(M, N_local, K, comm->world, 0);
  if (!workspace || workspace_bytes < need) return set_error(CFB200_ERR_WORKSPACE, "gemm_fp8_colpar needs %zu bytes of workspace", need);
  char* ws = reinterpret_cast<char*>(workspace);
  const size_t out_bytes = align256(M * N_local * 2);
  const bool p2p = comm->world > 1 && M > 1 && use_peer_loads(out_bytes, comm->world);
  int32_t rc;
  if (p2p) {
    rc = ensure_exchange(comm, out_bytes, (cudaStream_t)stream);
    if (rc) return rc;
  }
  void* slot = p2p ? exchange_slot(comm) : nullptr;
  rc = cfb200_gemm_fp8(A, a_scales, W_local, w_scale, M, N_local, K, slot ? slot : ws, 0, error_flag, stream);
  if (rc) return rc;
  if (slot) return pull_columns(comm, M, N_local, 2, C, layout, (cudaStream_t)stream);
  return gather_columns(comm, ws, M, N_local, 2, C, layout, ws + out_bytes, (cudaStream_t)stream);
}

// ---- GPTQ: token-parallel Hessian ---------------------------------------------------------------------------------------------
extern "C" int32_t cfb200_gptq_hessian_scaled(const void* X, size_t T, size_t K, float alpha, float* H, void* xt_workspace,
                                              size_t workspace_bytes, int32_t* error_flag, void* stream);

extern "C" int32_t cfb200_gptq_hessian_sharded(cfb200_comm* comm, const void* X_local, size_t T_local, size_t T_total, size_t K,
                                               float* H, void* xt_workspace, size_t workspace_bytes, int32_t* error_flag,
                                               void* stream) {
  CFB_CHECK_ARG(comm != nullptr, "NULL communicator");
  CFB_CHECK_ARG(T_total >= T_local && T_total > 0, "T_total must cover T_local");
  int32_t rc;
  if (T_local > 0) rc = cfb200_gptq_hessian_scaled(X_local, T_local, K, 1.0f / (float)T_total, H, xt_workspace, workspace_bytes, error_flag, stream);
  else rc = cudaMemsetAsync(H, 0, K * K * sizeof(float), (cudaStream_t)stream) == cudaSuccess ? CFB200_OK : set_error(CFB200_ERR_CUDA, "cudaMemsetAsync failed");
  if (rc) return rc;
  if (comm->world > 1) {
    const NcclApi* api;
    rc = nccl_api(&api);
    if (rc) return rc;
    CFB_NCCL(api, api->AllReduce(H, H, K * K, ncclFloat32, ncclSum, comm->nccl, (cudaStream_t)stream));
  }
  return CFB200_OK;
}
