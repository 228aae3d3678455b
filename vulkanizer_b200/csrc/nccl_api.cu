// libnccl.so.2: collectives between the ranks of one machine over NVLink / NVSwitch peer memory.
//
// Same exported surface as k0zi/Vulkanizer's src/nccl/nccl.cpp:497-753 (the subset declared in include/vkzb_nccl.h; the rest
// answers ncclInvalidUsage like src/nccl/nccl_stubs.cpp:30-36), rebuilt for a machine whose GPUs reach one another directly:
//
//   bootstrap   a POSIX shared-memory object named after the 128-bit token in ncclUniqueId (the reference's
//               UniqueId{magic, token[2]}, nccl.cpp:59-66, 503-509) holds one slot per rank; only ADDRESSES travel through it,
//               as CUDA IPC handles of the caller's buffers, posted per operation in a 4-deep ring;
//   data        every collective is "pull": after a barrier (all ranks' streams have reached the operation, so their send
//               buffers are final) a rank reads its peers' send buffers through the IPC mappings, with stream-ordered
//               cudaMemcpyAsync (copy engines, no SMs, so a gather overlaps a GEMM) or a reduction kernel, and a closing
//               barrier tells the peers their buffers are free again;
//   barriers    device side: each rank stores a sequence number into a flag word in every peer's arena
//               (st.release.sys over NVLink) and waits, bounded by %globaltimer, for its own flags to reach it. The
//               collective stays asynchronous on its stream. When two ranks share a GPU (kernels of different ranks may
//               not wait on one another on one device) the ranks meet on counters in the shared-memory object instead and
//               the call synchronises its stream, as the reference's does (nccl.cpp:338).
//
// Reductions accumulate floats in double and integers in 64 bits, in rank order (nccl.cpp:152-182): identical bits everywhere.
// Every wait is bounded: VKZB_NCCL_TIMEOUT_S seconds on the host (default 120), 20 s on the device; ncclCommAbort releases
// host waiters (nccl.cpp:554-557).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#define VKZB_HAVE_CUDA_TYPES
#include "../../include/vkzb_nccl.h"

namespace {

constexpr int kMaxRanks = 16;
constexpr uint32_t kMagic = 0x564B5A42u;
constexpr int kPostRing = 8;   // collective posts a rank may have outstanding before every peer has read the oldest
constexpr int kP2pRing = 16;   // sends a rank may have posted to one peer before that peer has read the oldest
constexpr int kMaxCustomOps = 16;

struct IdPayload {
    uint32_t magic, reserved;
    uint64_t token[2];
};
static_assert(sizeof(IdPayload) <= NCCL_UNIQUE_ID_BYTES, "id payload");

struct BufferPost {
    cudaIpcMemHandle_t handle;
    uint64_t base, offset;
};
struct OpPost {
    BufferPost send, recv;
    double premul;  // factor this rank's contribution is multiplied by (premultiplied sums; 1 otherwise)
    uint32_t bad;   // the rank could not describe its buffers: peers fail at once instead of waiting
};
struct P2pPost {
    BufferPost buffer;
    uint64_t bytes;
};
struct RankSlot {
    std::atomic<uint32_t> state;  // 0 empty, 1 published, 2 left
    int pid;
    char busId[32];
    BufferPost arenaPost;  // the flag arena: the allocation that holds it and its offset there
    uint64_t arenaRaw;
    std::atomic<uint64_t> postSeq;      // operations whose addresses are posted
    std::atomic<uint64_t> readSeq;      // operations whose peer posts this rank has read (the posters' flow control)
    std::atomic<uint64_t> hostBarrier;  // host-side barriers passed (ranks sharing a GPU)
    OpPost posts[kPostRing];
    // point to point, per destination rank: sends posted (addresses) and, for ranks that share a GPU, sends whose data is
    // final; per source rank: posts read, and receives completed (the sender may reuse its buffer)
    std::atomic<uint64_t> p2pPosted[kMaxRanks], p2pReady[kMaxRanks];
    std::atomic<uint64_t> p2pRead[kMaxRanks], p2pDone[kMaxRanks];
    P2pPost p2p[kMaxRanks][kP2pRing];
    // ncclCommSplit: this rank's (color, key) of split number splitSeq, and how many splits it has finished reading
    std::atomic<uint64_t> splitSeq, splitRead;
    int splitColor, splitKey;
};
struct Shared {
    std::atomic<uint32_t> abort;
    RankSlot ranks[kMaxRanks];
};

// Device memory of one rank that its peers map: flag words written by the peers, and a status word.
struct Arena {
    unsigned long long flags[kMaxRanks];     // barrier: written by peer p, sequence number of the barrier p has reached
    unsigned long long p2pReady[kMaxRanks];  // written by sender p: its sends to this rank whose data is final
    unsigned long long p2pDone[kMaxRanks];   // written by receiver p: sends of this rank to p that p has copied
    unsigned status;
};

enum OpKind { kAllGather, kBroadcast, kAllReduce, kReduceScatter, kReduce, kGather, kAllToAll, kBarrierOnly, kSend, kRecv };

}  // namespace

struct ncclComm {
    int rank = 0, nranks = 1, device = 0;
    Shared* shared = nullptr;
    std::string shmName;
    Arena* arena = nullptr;
    Arena* peerArena[kMaxRanks] = {};
    uint64_t peerArenaBase[kMaxRanks] = {}, peerArenaGeneration[kMaxRanks] = {};  // what was opened to reach peerArena[p] (other processes only)
    bool samePid[kMaxRanks] = {};
    bool hostSync = false;  // some ranks share a GPU
    uint64_t opSeq = 0, deviceBarrierSeq = 0, hostBarrierSeq = 0, splitCount = 0;
    uint64_t sendSeq[kMaxRanks] = {}, recvSeq[kMaxRanks] = {};  // point-to-point messages sent to / received from each rank
    uint64_t idToken[2] = {};                                   // of the unique id: children of ncclCommSplit derive theirs from it
    struct CustomOp {
        bool live = false;
        double factor = 1.0;
        const void* devicePointer = nullptr;  // ncclScalarDevice: read when the collective is issued
        ncclDataType_t type = ncclFloat32;
    } customOps[kMaxCustomOps];
    struct Mapping {
        cudaIpcMemHandle_t handle;
        void* local;
        uint64_t generation;  // of the process-wide mapping this one uses
    };
    std::map<std::pair<int, uint64_t>, Mapping> mappings;  // (peer, remote base) -> local mapping
    std::string lastError;
    std::atomic<bool> aborted{false};
};

namespace {

thread_local int t_groupDepth = 0;

struct Op {
    ncclComm* comm;
    int kind;
    const void* send;
    void* recv;
    size_t count;
    ncclDataType_t type;
    ncclRedOp_t op;
    int root;
    cudaStream_t stream;
    uint64_t seq = 0;
    const char* peerSend[kMaxRanks] = {};
    char* peerRecv[kMaxRanks] = {};
    double premul[kMaxRanks] = {};  // per rank, for premultiplied sums
    bool scaled = false;
    int peer = -1;                  // kSend / kRecv
    uint64_t p2pSeq = 0;
};
thread_local std::vector<Op> t_queue;

// How long a device-side wait may last before it gives up (VKZB_NCCL_DEVICE_WAIT_MS; default 20 s).
unsigned long long deviceWaitNs() {
    static const unsigned long long ns = [] {
        const char* v = std::getenv("VKZB_NCCL_DEVICE_WAIT_MS");
        const double ms = v ? std::atof(v) : 0;
        return ms > 0 ? (unsigned long long)(ms * 1e6) : 20000000000ull;
    }();
    return ns;
}

double timeoutSeconds() {
    static const double s = [] {
        const char* v = std::getenv("VKZB_NCCL_TIMEOUT_S");
        const double d = v ? std::atof(v) : 0;
        return d > 0 ? d : 120.0;
    }();
    return s;
}

size_t typeSize(ncclDataType_t t) {
    switch (t) {
    case ncclInt8: case ncclUint8: case ncclFloat8e4m3: case ncclFloat8e5m2: return 1;
    case ncclFloat16: case ncclBfloat16: return 2;
    case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
    case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
    default: return 0;
    }
}

ncclResult_t fail(ncclComm* c, ncclResult_t r, const std::string& what) {
    if (c) c->lastError = what;
    if (std::getenv("VKZB_LOG")) std::fprintf(stderr, "vkzb nccl: %s\n", what.c_str());
    return r;
}

// Polls `ready` with a back-off until it holds, the communicator is aborted, or the time is up.
template <class F>
ncclResult_t hostWait(ncclComm* c, F ready, const char* what) {
    const auto start = std::chrono::steady_clock::now();
    for (unsigned spins = 0;; ++spins) {
        if (ready()) return ncclSuccess;
        if (c->aborted.load() || c->shared->abort.load()) return fail(c, ncclRemoteError, std::string("aborted while waiting for ") + what);
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count() > timeoutSeconds())
            return fail(c, ncclRemoteError, std::string("timed out waiting for ") + what);
        if (spins < 2000) std::this_thread::yield();
        else std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

// A scalar of an NCCL data type as a double (premultiplied sums).
double scalarValue(const void* p, ncclDataType_t t) {
    switch (t) {
    case ncclInt8: return double(*static_cast<const signed char*>(p));
    case ncclUint8: return double(*static_cast<const unsigned char*>(p));
    case ncclInt32: return double(*static_cast<const int*>(p));
    case ncclUint32: return double(*static_cast<const unsigned*>(p));
    case ncclInt64: return double(*static_cast<const long long*>(p));
    case ncclUint64: return double(*static_cast<const unsigned long long*>(p));
    case ncclFloat16: return double(__half2float(*static_cast<const __half*>(p)));
    case ncclBfloat16: return double(__bfloat162float(*static_cast<const __nv_bfloat16*>(p)));
    case ncclFloat32: return double(*static_cast<const float*>(p));
    case ncclFloat64: return *static_cast<const double*>(p);
    default: return 1.0;
    }
}

// ---- device side ----------------------------------------------------------------------------------------------------

struct FlagTable {
    unsigned long long* peer[kMaxRanks];  // peer p's flag word for this rank
};

__global__ void barrierKernel(FlagTable peers, unsigned long long* mine, unsigned* status, int me, int n, unsigned long long seq,
                              unsigned long long waitNs) {
    const int p = threadIdx.x;
    if (p >= n || p == me) return;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(peers.peer[p]), "l"(seq) : "memory");
    unsigned long long start;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine + p) : "memory");
        if (v >= seq) return;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - start > waitNs) {
            atomicExch(status, 1u + unsigned(p));  // peer p never arrived
            return;
        }
        __nanosleep(200);
    }
}

// Point to point between ranks on different GPUs: one thread tells a peer "my message number seq is ready / is copied" ...
__global__ void signalKernel(unsigned long long* flag, unsigned long long seq) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(seq) : "memory");
}
// ... and one waits, bounded, for the peer's word to reach seq.
__global__ void waitKernel(const unsigned long long* flag, unsigned long long seq, unsigned* status, unsigned code, unsigned long long waitNs) {
    unsigned long long start;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
        if (v >= seq) return;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - start > waitNs) {
            atomicExch(status, code);
            return;
        }
        __nanosleep(200);
    }
}

struct SourceTable {
    const void* src[kMaxRanks];
    double scale[kMaxRanks];  // premultiplied sums: contribution r is multiplied by scale[r] before it is added
    int scaled;
};

template <typename T> struct AccOf { using type = double; };
template <> struct AccOf<signed char> { using type = long long; };
template <> struct AccOf<unsigned char> { using type = unsigned long long; };
template <> struct AccOf<int> { using type = long long; };
template <> struct AccOf<unsigned> { using type = unsigned long long; };
template <> struct AccOf<long long> { using type = long long; };
template <> struct AccOf<unsigned long long> { using type = unsigned long long; };

template <typename A, typename T> __device__ __forceinline__ A widen(T v) { return A(v); }
template <> __device__ __forceinline__ double widen<double, __half>(__half v) { return double(__half2float(v)); }
template <> __device__ __forceinline__ double widen<double, __nv_bfloat16>(__nv_bfloat16 v) { return double(__bfloat162float(v)); }
template <typename T, typename A> __device__ __forceinline__ T narrow(A v) { return T(v); }
template <> __device__ __forceinline__ __half narrow<__half, double>(double v) { return __float2half_rn(float(v)); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, double>(double v) { return __float2bfloat16_rn(float(v)); }

// out[i] = reduction over ranks, in rank order, of src[r][i]; every rank that runs it gets the same bits.
template <typename T>
__global__ void reduceKernel(T* out, SourceTable table, size_t n, int nranks, int op) {
    using A = typename AccOf<T>::type;
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        A acc = widen<A, T>(static_cast<const T*>(table.src[0])[i]);
        if (table.scaled) acc = acc * A(table.scale[0]);
        for (int r = 1; r < nranks; ++r) {
            A v = widen<A, T>(static_cast<const T*>(table.src[r])[i]);
            if (table.scaled) v = v * A(table.scale[r]);
            if (op == ncclProd) acc = acc * v;
            else if (op == ncclMax) acc = v > acc ? v : acc;
            else if (op == ncclMin) acc = v < acc ? v : acc;
            else acc = acc + v;
        }
        if (op == ncclAvg) acc = acc / A(nranks);
        out[i] = narrow<T, A>(acc);
    }
}

cudaError_t launchReduce(void* out, const SourceTable& t, size_t n, int nranks, ncclDataType_t type, int op, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    const int threads = 256;
    const unsigned blocks = unsigned(std::min<size_t>((n + threads - 1) / threads, 1024));
    switch (type) {
    case ncclInt8: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<signed char*>(out), t, n, nranks, op); break;
    case ncclUint8: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<unsigned char*>(out), t, n, nranks, op); break;
    case ncclInt32: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<int*>(out), t, n, nranks, op); break;
    case ncclUint32: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<unsigned*>(out), t, n, nranks, op); break;
    case ncclInt64: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<long long*>(out), t, n, nranks, op); break;
    case ncclUint64: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<unsigned long long*>(out), t, n, nranks, op); break;
    case ncclFloat16: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<__half*>(out), t, n, nranks, op); break;
    case ncclBfloat16: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<__nv_bfloat16*>(out), t, n, nranks, op); break;
    case ncclFloat32: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<float*>(out), t, n, nranks, op); break;
    case ncclFloat64: reduceKernel<<<blocks, threads, 0, s>>>(static_cast<double*>(out), t, n, nranks, op); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// ---- addresses -------------------------------------------------------------------------------------------------------

using AddressRangeFn = int (*)(unsigned long long*, size_t*, unsigned long long);

AddressRangeFn addressRange() {
    static const AddressRangeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<AddressRangeFn>(p);
    }();
    return fn;
}

// The IPC handle of the allocation that holds `ptr`, and ptr's offset in it.
bool describeBuffer(const void* ptr, BufferPost& out) {
    std::memset(&out, 0, sizeof out);
    if (!ptr) return true;
    unsigned long long base = 0;
    size_t size = 0;
    if (!addressRange() || addressRange()(&base, &size, reinterpret_cast<unsigned long long>(ptr)) != 0) return false;
    out.base = base;
    out.offset = reinterpret_cast<unsigned long long>(ptr) - base;
    return cudaIpcGetMemHandle(&out.handle, reinterpret_cast<void*>(base)) == cudaSuccess;
}

// CUDA maps an allocation of another process into this one only once at a time, and the handles it gives out do not name
// allocations one to one: small cudaMalloc requests share blocks, and two buffers of one block come with different handles
// of which only one can be open ("resource already mapped" for the second). So what this process has opened is kept
// process-wide, keyed by the owner's process and the allocation's base address there, and counted: a second buffer of a
// block that is already open reuses the mapping, whichever communicator asks.
struct IpcKey {
    int device, pid;
    uint64_t base;
    bool operator<(const IpcKey& o) const { return device != o.device ? device < o.device : pid != o.pid ? pid < o.pid : base < o.base; }
};
struct IpcOpened {
    cudaIpcMemHandle_t handle;
    void* local;
    int users;
    uint64_t generation;
};
std::mutex g_ipcMutex;
std::map<IpcKey, IpcOpened> g_ipcOpened;
uint64_t g_ipcGeneration = 0;

IpcKey ipcKeyOf(int pid, uint64_t base) {
    IpcKey k{};
    cudaGetDevice(&k.device);
    k.pid = pid, k.base = base;
    return k;
}

// The local address of the allocation of process `pid` that starts at `base` there. `generation` identifies the mapping for
// ipcRelease (a later allocation at the same address is a different mapping).
void* ipcAcquire(int pid, uint64_t base, const cudaIpcMemHandle_t& handle, uint64_t& generation) {
    const IpcKey key = ipcKeyOf(pid, base);
    std::lock_guard<std::mutex> lock(g_ipcMutex);
    auto it = g_ipcOpened.find(key);
    if (it != g_ipcOpened.end() && std::memcmp(&it->second.handle, &handle, sizeof handle) == 0) {
        ++it->second.users;
        generation = it->second.generation;
        return it->second.local;
    }
    void* local = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&local, handle, cudaIpcMemLazyEnablePeerAccess);
    if (e == cudaSuccess) {
        if (it != g_ipcOpened.end()) {  // the owner freed the old allocation and got this address again: the old mapping is dead
            cudaIpcCloseMemHandle(it->second.local);
            g_ipcOpened.erase(it);
        }
        generation = ++g_ipcGeneration;
        g_ipcOpened.emplace(key, IpcOpened{handle, local, 1, generation});
        return local;
    }
    cudaGetLastError();
    if (e == cudaErrorAlreadyMapped && it != g_ipcOpened.end()) {  // another handle of the block that is open already
        ++it->second.users;
        generation = it->second.generation;
        return it->second.local;
    }
    if (std::getenv("VKZB_LOG")) std::fprintf(stderr, "vkzb nccl: cudaIpcOpenMemHandle: %s (%zu allocations open)\n", cudaGetErrorString(e), g_ipcOpened.size());
    return nullptr;
}

void ipcRelease(int pid, uint64_t base, uint64_t generation) {
    const IpcKey key = ipcKeyOf(pid, base);
    std::lock_guard<std::mutex> lock(g_ipcMutex);
    auto it = g_ipcOpened.find(key);
    if (it == g_ipcOpened.end() || it->second.generation != generation) return;
    if (--it->second.users == 0) {
        cudaIpcCloseMemHandle(it->second.local);
        g_ipcOpened.erase(it);
    }
}

// Local address of a peer's posted buffer: the raw pointer inside one process, an IPC mapping across processes.
void* mapPeerBuffer(ncclComm* c, int peer, const BufferPost& post) {
    if (!post.base) return nullptr;
    if (c->samePid[peer]) return reinterpret_cast<void*>(post.base + post.offset);
    const int pid = c->shared->ranks[peer].pid;
    const auto key = std::make_pair(peer, post.base);
    auto it = c->mappings.find(key);
    if (it != c->mappings.end() && std::memcmp(&it->second.handle, &post.handle, sizeof post.handle) != 0) {
        ipcRelease(pid, post.base, it->second.generation);  // another buffer of the block, or the address was freed and allocated again
        c->mappings.erase(it);
        it = c->mappings.end();
    }
    if (it == c->mappings.end()) {
        uint64_t generation = 0;
        void* local = ipcAcquire(pid, post.base, post.handle, generation);
        if (!local) return nullptr;
        it = c->mappings.emplace(key, ncclComm::Mapping{post.handle, local, generation}).first;
    }
    return static_cast<char*>(it->second.local) + post.offset;
}

// ---- barriers ---------------------------------------------------------------------------------------------------------

ncclResult_t barrier(std::vector<Op*>& ops) {
    // device side where every rank has its own GPU: asynchronous on the stream
    for (Op* o : ops) {
        ncclComm* c = o->comm;
        if (c->hostSync || c->nranks == 1) continue;
        FlagTable t{};
        for (int p = 0; p < c->nranks; ++p) t.peer[p] = p == c->rank ? nullptr : &c->peerArena[p]->flags[c->rank];
        barrierKernel<<<1, 32, 0, o->stream>>>(t, c->arena->flags, &c->arena->status, c->rank, c->nranks, ++c->deviceBarrierSeq, deviceWaitNs());
        if (cudaGetLastError() != cudaSuccess) return fail(c, ncclUnhandledCudaError, "barrier kernel launch failed");
    }
    // host side where ranks share a GPU: drain the streams, publish, then wait for the peers
    for (Op* o : ops) {
        ncclComm* c = o->comm;
        if (!c->hostSync || c->nranks == 1) continue;
        if (cudaStreamSynchronize(o->stream) != cudaSuccess) return fail(c, ncclUnhandledCudaError, "stream synchronize failed");
        c->shared->ranks[c->rank].hostBarrier.store(++c->hostBarrierSeq, std::memory_order_release);
    }
    for (Op* o : ops) {
        ncclComm* c = o->comm;
        if (!c->hostSync || c->nranks == 1) continue;
        const uint64_t want = c->hostBarrierSeq;
        const ncclResult_t r = hostWait(c, [&] {
            for (int p = 0; p < c->nranks; ++p)
                if (c->shared->ranks[p].hostBarrier.load(std::memory_order_acquire) < want) return false;
            return true;
        }, "the other ranks at a barrier");
        if (r != ncclSuccess) return r;
    }
    return ncclSuccess;
}

// ---- the collectives, as one or two rounds of pulls --------------------------------------------------------------------

cudaError_t copyAsync(void* dst, const void* src, size_t bytes, cudaStream_t s) {
    if (bytes == 0 || dst == src) return cudaSuccess;
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s);
}

void sliceOf(size_t count, int nranks, int r, size_t& first, size_t& len) {
    const size_t per = (count + nranks - 1) / nranks;
    first = std::min(count, per * size_t(r));
    len = std::min(count, first + per) - first;
}

bool needsSecondRound(const Op& o) { return o.kind == kAllReduce; }

ncclResult_t runRound(Op& o, int round) {
    ncclComm* c = o.comm;
    const int n = c->nranks, me = c->rank;
    const size_t es = typeSize(o.type), bytes = o.count * es;
    cudaError_t e = cudaSuccess;
    const auto local = [&](int p) { return p == me; };
    switch (o.kind) {
    case kAllGather:
        // start with the next rank so that the ranks do not all read from rank 0 at the same moment
        for (int i = 0; i < n && e == cudaSuccess; ++i) {
            const int p = (me + 1 + i) % n;
            e = copyAsync(static_cast<char*>(o.recv) + size_t(p) * bytes, local(p) ? static_cast<const char*>(o.send) : o.peerSend[p], bytes, o.stream);
        }
        break;
    case kBroadcast:
        e = copyAsync(o.recv, local(o.root) ? static_cast<const char*>(o.send) : o.peerSend[o.root], bytes, o.stream);
        break;
    case kGather:
        if (me == o.root)
            for (int i = 0; i < n && e == cudaSuccess; ++i) {
                const int p = (me + 1 + i) % n;
                e = copyAsync(static_cast<char*>(o.recv) + size_t(p) * bytes, local(p) ? static_cast<const char*>(o.send) : o.peerSend[p], bytes, o.stream);
            }
        break;
    case kAllToAll:
        for (int i = 0; i < n && e == cudaSuccess; ++i) {
            const int p = (me + 1 + i) % n;
            const char* src = (local(p) ? static_cast<const char*>(o.send) : o.peerSend[p]) + size_t(me) * bytes;
            e = copyAsync(static_cast<char*>(o.recv) + size_t(p) * bytes, src, bytes, o.stream);
        }
        break;
    case kBarrierOnly:
    case kSend:
    case kRecv:
        break;
    case kReduce:
    case kReduceScatter: {
        if (o.kind == kReduce && me != o.root) break;
        SourceTable t{};
        const size_t skip = o.kind == kReduceScatter ? size_t(me) * bytes : 0;  // rank r keeps block r of the reduction
        for (int p = 0; p < n; ++p) t.src[p] = (local(p) ? static_cast<const char*>(o.send) : o.peerSend[p]) + skip, t.scale[p] = o.premul[p];
        t.scaled = o.scaled;
        e = launchReduce(o.recv, t, o.count, n, o.type, o.scaled ? ncclSum : o.op, o.stream);
        break;
    }
    case kAllReduce: {
        // round 0: this rank reduces its slice of every rank's send buffer into its own receive buffer (no rank reads the
        // slice another one writes, so send == recv is safe); round 1: it pulls the other slices from their owners.
        if (round == 0) {
            size_t first, len;
            sliceOf(o.count, n, me, first, len);
            SourceTable t{};
            for (int p = 0; p < n; ++p) t.src[p] = (local(p) ? static_cast<const char*>(o.send) : o.peerSend[p]) + first * es, t.scale[p] = o.premul[p];
            t.scaled = o.scaled;
            e = launchReduce(static_cast<char*>(o.recv) + first * es, t, len, n, o.type, o.scaled ? ncclSum : o.op, o.stream);
        } else {
            for (int i = 0; i + 1 < n && e == cudaSuccess; ++i) {
                const int p = (me + 1 + i) % n;
                size_t first, len;
                sliceOf(o.count, n, p, first, len);
                e = copyAsync(static_cast<char*>(o.recv) + first * es, o.peerRecv[p] + first * es, len * es, o.stream);
            }
        }
        break;
    }
    }
    return e == cudaSuccess ? ncclSuccess : fail(c, ncclUnhandledCudaError, std::string("data movement failed: ") + cudaGetErrorString(e));
}

// ---- point to point ---------------------------------------------------------------------------------------------------------
//
// A send posts its buffer's address for the receiver (a ring per ordered pair, matched by sequence number like the
// reference's, nccl.cpp:340-347) and tells it when the data is final; the receiver pulls the bytes and tells the sender when
// it has them, which is when the send completes on its stream. Between GPUs the two notices are flag words in the peers'
// arenas, written and awaited by one-thread kernels on the operations' streams; ranks that share a GPU use counters in the
// shared-memory object and synchronise their streams. Within a group every "data is final" notice goes out before anything
// waits, so a ring of sends and receives, or an exchange with every peer, cannot wait on itself.
ncclResult_t runPointToPoint(std::vector<Op*>& ops) {
    std::vector<Op*> sends, recvs;
    for (Op* o : ops) (o->kind == kSend ? sends : recvs).push_back(o);
    // 1. post the send buffers' addresses
    std::vector<std::pair<const void*, size_t>> toSelf;  // sends of a rank to itself, matched to its receives in order
    size_t selfTaken = 0;
    for (Op* o : sends) {
        ncclComm* c = o->comm;
        cudaSetDevice(c->device);
        if (o->peer == c->rank) {
            toSelf.emplace_back(o->send, o->count * typeSize(o->type));
            continue;
        }
        RankSlot& slot = c->shared->ranks[c->rank];
        o->p2pSeq = ++c->sendSeq[o->peer];
        if (o->p2pSeq > kP2pRing) {  // the slot about to be reused must have been read by the receiver
            const uint64_t need = o->p2pSeq - kP2pRing;
            const ncclResult_t r = hostWait(c, [&] { return c->shared->ranks[o->peer].p2pRead[c->rank].load(std::memory_order_acquire) >= need; },
                                            "a peer to take earlier point-to-point messages");
            if (r != ncclSuccess) return r;
        }
        P2pPost& post = slot.p2p[o->peer][o->p2pSeq % kP2pRing];
        post.bytes = o->count * typeSize(o->type);
        if (!describeBuffer(o->send, post.buffer)) post.bytes = ~0ull;  // the receiver fails at once instead of waiting
        slot.p2pPosted[o->peer].store(o->p2pSeq, std::memory_order_release);
        if (post.bytes == ~0ull) return fail(c, ncclInvalidArgument, "the send buffer is not device memory that can be shared with the other ranks");
    }
    // 2. "my data is final": a flag store on the stream, or (shared GPU) a host counter once the stream has drained
    for (Op* o : sends) {
        ncclComm* c = o->comm;
        if (o->peer == c->rank) continue;
        cudaSetDevice(c->device);
        if (c->hostSync) {
            if (cudaStreamSynchronize(o->stream) != cudaSuccess) return fail(c, ncclUnhandledCudaError, "stream synchronize failed");
            c->shared->ranks[c->rank].p2pReady[o->peer].store(o->p2pSeq, std::memory_order_release);
        } else {
            signalKernel<<<1, 1, 0, o->stream>>>(&c->peerArena[o->peer]->p2pReady[c->rank], o->p2pSeq);
            if (cudaGetLastError() != cudaSuccess) return fail(c, ncclUnhandledCudaError, "signal kernel launch failed");
        }
    }
    // 3. receives: find the matching post, wait for the data, pull it, say so
    for (Op* o : recvs) {
        ncclComm* c = o->comm;
        cudaSetDevice(c->device);
        const size_t bytes = o->count * typeSize(o->type);
        if (o->peer == c->rank) {
            if (selfTaken >= toSelf.size()) return fail(c, ncclInvalidUsage, "a receive from this rank itself needs a send to itself in the same group");
            const auto& from = toSelf[selfTaken++];
            if (from.second != bytes) return fail(c, ncclInvalidArgument, "send and receive sizes differ");
            if (copyAsync(o->recv, from.first, bytes, o->stream) != cudaSuccess) return fail(c, ncclUnhandledCudaError, "copy failed");
            continue;
        }
        o->p2pSeq = ++c->recvSeq[o->peer];
        RankSlot& theirs = c->shared->ranks[o->peer];
        ncclResult_t r = hostWait(c, [&] { return theirs.p2pPosted[c->rank].load(std::memory_order_acquire) >= o->p2pSeq; }, "the matching send to be posted");
        if (r != ncclSuccess) return r;
        const P2pPost post = theirs.p2p[c->rank][o->p2pSeq % kP2pRing];
        c->shared->ranks[c->rank].p2pRead[o->peer].store(o->p2pSeq, std::memory_order_release);
        if (post.bytes == ~0ull) return fail(c, ncclRemoteError, "the sender could not share its buffer");
        if (post.bytes != bytes) return fail(c, ncclInvalidArgument, "send and receive sizes differ");
        const void* src = mapPeerBuffer(c, o->peer, post.buffer);
        if (!src && bytes) return fail(c, ncclUnhandledCudaError, "could not map the sender's buffer (cudaIpcOpenMemHandle)");
        if (c->hostSync) {
            r = hostWait(c, [&] { return theirs.p2pReady[c->rank].load(std::memory_order_acquire) >= o->p2pSeq; }, "the sender's data");
            if (r != ncclSuccess) return r;
            if (copyAsync(o->recv, src, bytes, o->stream) != cudaSuccess || cudaStreamSynchronize(o->stream) != cudaSuccess)
                return fail(c, ncclUnhandledCudaError, "copy failed");
            c->shared->ranks[c->rank].p2pDone[o->peer].store(o->p2pSeq, std::memory_order_release);
        } else {
            waitKernel<<<1, 1, 0, o->stream>>>(&c->arena->p2pReady[o->peer], o->p2pSeq, &c->arena->status, 101u + unsigned(o->peer), deviceWaitNs());
            if (cudaGetLastError() != cudaSuccess || copyAsync(o->recv, src, bytes, o->stream) != cudaSuccess)
                return fail(c, ncclUnhandledCudaError, "receive failed");
            signalKernel<<<1, 1, 0, o->stream>>>(&c->peerArena[o->peer]->p2pDone[c->rank], o->p2pSeq);
            if (cudaGetLastError() != cudaSuccess) return fail(c, ncclUnhandledCudaError, "signal kernel launch failed");
        }
    }
    if (selfTaken != toSelf.size()) return fail(sends.front()->comm, ncclInvalidUsage, "a send to this rank itself needs a receive from itself in the same group");
    // 4. a send is complete when the receiver has the data
    for (Op* o : sends) {
        ncclComm* c = o->comm;
        if (o->peer == c->rank) continue;
        cudaSetDevice(c->device);
        if (c->hostSync) {
            const ncclResult_t r = hostWait(c, [&] { return c->shared->ranks[o->peer].p2pDone[c->rank].load(std::memory_order_acquire) >= o->p2pSeq; },
                                            "the receiver to take a message");
            if (r != ncclSuccess) return r;
        } else {
            waitKernel<<<1, 1, 0, o->stream>>>(&c->arena->p2pDone[o->peer], o->p2pSeq, &c->arena->status, 201u + unsigned(o->peer), deviceWaitNs());
            if (cudaGetLastError() != cudaSuccess) return fail(c, ncclUnhandledCudaError, "wait kernel launch failed");
        }
    }
    return ncclSuccess;
}

// ---- collectives ------------------------------------------------------------------------------------------------------------

// One batch: at most kPostRing operations per communicator, so no operation of the batch can overwrite the posted addresses
// of another one that a peer has yet to read.
ncclResult_t executeCollectives(std::vector<Op*>& ops) {
    // 1. every operation posts its buffers' addresses
    for (Op* op : ops) {
        Op& o = *op;
        ncclComm* c = o.comm;
        cudaSetDevice(c->device);
        o.seq = ++c->opSeq;
        for (int p = 0; p < c->nranks; ++p) o.premul[p] = 1.0;
        double myFactor = 1.0;
        if (int(o.op) >= int(ncclNumOps)) {  // a premultiplied sum created by ncclRedOpCreatePreMulSum
            const ncclComm::CustomOp& custom = c->customOps[int(o.op) - int(ncclNumOps)];
            myFactor = custom.factor;
            if (custom.devicePointer) {  // a scalar in device memory is read when the collective is issued, after the stream's earlier work
                unsigned char raw[8] = {};
                if (cudaStreamSynchronize(o.stream) != cudaSuccess || cudaMemcpy(raw, custom.devicePointer, typeSize(custom.type), cudaMemcpyDeviceToHost) != cudaSuccess)
                    return fail(c, ncclUnhandledCudaError, "could not read the scalar of a premultiplied sum");
                myFactor = scalarValue(raw, custom.type);
            }
            o.scaled = true;
            o.premul[c->rank] = myFactor;
        }
        if (c->nranks == 1) continue;
        RankSlot& slot = c->shared->ranks[c->rank];
        if (o.seq > kPostRing) {  // flow control: the slot about to be rewritten was read by every peer
            const uint64_t need = o.seq - kPostRing;
            const ncclResult_t r = hostWait(c, [&] {
                for (int p = 0; p < c->nranks; ++p)
                    if (p != c->rank && c->shared->ranks[p].readSeq.load(std::memory_order_acquire) < need) return false;
                return true;
            }, "the other ranks to finish reading an earlier collective's addresses");
            if (r != ncclSuccess) return r;
        }
        OpPost& post = slot.posts[o.seq % kPostRing];
        post.premul = myFactor;
        post.bad = !describeBuffer(o.send, post.send) || !describeBuffer(o.recv, post.recv);
        const bool bad = post.bad != 0;
        slot.postSeq.store(o.seq, std::memory_order_release);  // published even when bad, so that the peers do not wait for it
        if (bad) return fail(c, ncclInvalidArgument, "a buffer is not device memory that can be shared with the other ranks (cudaMalloc memory is)");
    }
    // 2. ... and maps what the peers posted
    for (Op* op : ops) {
        Op& o = *op;
        ncclComm* c = o.comm;
        if (c->nranks == 1) continue;
        cudaSetDevice(c->device);
        const ncclResult_t r = hostWait(c, [&] {
            for (int p = 0; p < c->nranks; ++p)
                if (c->shared->ranks[p].postSeq.load(std::memory_order_acquire) < o.seq) return false;
            return true;
        }, "the other ranks to enter the collective");
        if (r != ncclSuccess) return r;
        ncclResult_t result = ncclSuccess;
        for (int p = 0; p < c->nranks && result == ncclSuccess; ++p) {
            if (p == c->rank) continue;
            const OpPost post = c->shared->ranks[p].posts[o.seq % kPostRing];
            if (post.bad) {
                result = fail(c, ncclRemoteError, "another rank could not share its buffers");
                break;
            }
            o.premul[p] = post.premul;
            o.peerSend[p] = static_cast<const char*>(mapPeerBuffer(c, p, post.send));
            o.peerRecv[p] = static_cast<char*>(mapPeerBuffer(c, p, post.recv));
            const bool needSend = !(o.kind == kBroadcast && p != o.root) && !((o.kind == kGather || o.kind == kReduce) && c->rank != o.root);
            if ((needSend && post.send.base && !o.peerSend[p]) || (o.kind == kAllReduce && !o.peerRecv[p]))
                result = fail(c, ncclUnhandledCudaError, "could not map a peer's buffer (cudaIpcOpenMemHandle)");
        }
        c->shared->ranks[c->rank].readSeq.store(o.seq, std::memory_order_release);  // read (even if unusable): the slots may be reused
        if (result != ncclSuccess) return result;
    }
    // 3. barrier, pulls, (barrier, pulls,) barrier
    std::vector<Op*> second;
    for (Op* o : ops)
        if (needsSecondRound(*o)) second.push_back(o);
    ncclResult_t r = barrier(ops);
    for (Op* o : ops) {
        if (r != ncclSuccess) return r;
        cudaSetDevice(o->comm->device);
        r = runRound(*o, 0);
    }
    if (r == ncclSuccess && !second.empty()) {
        r = barrier(second);
        for (Op* o : second) {
            if (r != ncclSuccess) return r;
            cudaSetDevice(o->comm->device);
            r = runRound(*o, 1);
        }
    }
    if (r == ncclSuccess) {
        std::vector<Op*> closing;
        for (Op* o : ops)
            if (o->kind != kBarrierOnly) closing.push_back(o);
        r = barrier(closing);
    }
    return r;
}

// Everything one ncclGroupEnd (or one ungrouped call) starts: the collectives in batches that respect the posting ring, the
// sends and receives together.
ncclResult_t execute(std::vector<Op>& ops) {
    std::vector<Op*> p2p, batch;
    std::map<ncclComm*, int> inBatch;
    const auto flush = [&]() {
        const ncclResult_t r = batch.empty() ? ncclSuccess : executeCollectives(batch);
        batch.clear();
        inBatch.clear();
        return r;
    };
    for (Op& o : ops) {
        if (o.comm->aborted.load()) return fail(o.comm, ncclInvalidUsage, "communicator was aborted");
        if (o.kind == kSend || o.kind == kRecv) {
            p2p.push_back(&o);
            continue;
        }
        if (inBatch[o.comm] == kPostRing)
            if (const ncclResult_t r = flush(); r != ncclSuccess) return r;
        batch.push_back(&o);
        ++inBatch[o.comm];
    }
    if (const ncclResult_t r = flush(); r != ncclSuccess) return r;
    return p2p.empty() ? ncclSuccess : runPointToPoint(p2p);
}

ncclResult_t submit(Op op) {
    if (!op.comm) return ncclInvalidArgument;
    const bool reduces = op.kind == kAllReduce || op.kind == kReduce || op.kind == kReduceScatter;
    if (op.kind != kBarrierOnly && (typeSize(op.type) == 0 || (!op.recv && op.count && !(op.kind == kReduce || op.kind == kGather || op.kind == kSend))))
        return fail(op.comm, ncclInvalidArgument, "bad datatype or null buffer");
    if ((op.kind == kBroadcast || op.kind == kReduce || op.kind == kGather) && (op.root < 0 || op.root >= op.comm->nranks))
        return fail(op.comm, ncclInvalidArgument, "root out of range");
    if ((op.kind == kSend || op.kind == kRecv) && (op.peer < 0 || op.peer >= op.comm->nranks))
        return fail(op.comm, ncclInvalidArgument, "peer out of range");
    if (reduces && int(op.op) >= int(ncclNumOps)) {
        const int index = int(op.op) - int(ncclNumOps);
        if (index >= kMaxCustomOps || !op.comm->customOps[index].live) return fail(op.comm, ncclInvalidArgument, "unknown reduction operator");
    } else if (reduces && int(op.op) < 0) {
        return fail(op.comm, ncclInvalidArgument, "unknown reduction operator");
    }
    if (t_groupDepth > 0) {
        t_queue.push_back(op);
        return ncclSuccess;
    }
    std::vector<Op> one{op};
    int prev = 0;
    cudaGetDevice(&prev);
    const ncclResult_t r = execute(one);
    cudaSetDevice(prev);
    return r;
}

std::string shmNameOf(const IdPayload& id) {
    char name[80];
    std::snprintf(name, sizeof name, "/vkzb-nccl-%016llx%016llx", (unsigned long long)id.token[0], (unsigned long long)id.token[1]);
    return name;
}

// Flag arenas come from one block per device and process, exported once: CUDA maps an allocation into a peer process only
// once at a time, and small cudaMalloc requests share blocks, so a second communicator of the same processes (ncclCommSplit,
// or simply another ncclCommInitRank) whose arena had landed in a block its peers already hold open could not be mapped
// ("resource already mapped"). With every arena in the one block and every post carrying the block's one handle, the peers
// open it once and count its users.
constexpr size_t kArenaSlotBytes = 1024, kArenaPoolBytes = size_t(2) << 20;
static_assert(sizeof(Arena) <= kArenaSlotBytes, "arena slot");
struct ArenaPool {
    char* base = nullptr;
    cudaIpcMemHandle_t handle{};
    std::vector<bool> taken;
};
std::mutex g_arenaMutex;
ArenaPool g_arenaPools[64];

Arena* arenaTake(int device, BufferPost& post) {
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_arenaMutex);
    ArenaPool& pool = g_arenaPools[device];
    if (!pool.base) {
        void* block = nullptr;
        if (cudaMalloc(&block, kArenaPoolBytes) != cudaSuccess || cudaIpcGetMemHandle(&pool.handle, block) != cudaSuccess) {
            cudaGetLastError();
            if (block) cudaFree(block);
            return nullptr;
        }
        pool.base = static_cast<char*>(block);
        pool.taken.assign(kArenaPoolBytes / kArenaSlotBytes, false);
    }
    for (size_t i = 0; i < pool.taken.size(); ++i) {
        if (pool.taken[i]) continue;
        char* slot = pool.base + i * kArenaSlotBytes;
        if (cudaMemset(slot, 0, kArenaSlotBytes) != cudaSuccess) return nullptr;
        pool.taken[i] = true;
        std::memset(&post, 0, sizeof post);
        post.handle = pool.handle;
        post.base = reinterpret_cast<uint64_t>(pool.base);
        post.offset = i * kArenaSlotBytes;
        return reinterpret_cast<Arena*>(slot);
    }
    return nullptr;
}

void arenaGive(int device, Arena* arena) {
    if (!arena || device < 0 || device >= 64) return;
    std::lock_guard<std::mutex> lock(g_arenaMutex);
    ArenaPool& pool = g_arenaPools[device];
    if (pool.base) pool.taken[size_t(reinterpret_cast<char*>(arena) - pool.base) / kArenaSlotBytes] = false;
}

// Gives back what a communicator holds on this side (mappings, arena, the shared-memory view). `announce`: tell the peers
// that this rank has left (and remove the shared-memory object's name once every rank has).
void release(ncclComm* c, bool announce) {
    if (c->shared) {
        for (auto& m : c->mappings) ipcRelease(c->shared->ranks[m.first.first].pid, m.first.second, m.second.generation);
        for (int p = 0; p < c->nranks; ++p)
            if (p != c->rank && c->peerArena[p] && !c->samePid[p])
                ipcRelease(c->shared->ranks[p].pid, c->peerArenaBase[p], c->peerArenaGeneration[p]), c->peerArena[p] = nullptr;
    }
    c->mappings.clear();
    if (c->shared) {
        if (announce) {
            c->shared->ranks[c->rank].state.store(2, std::memory_order_release);
            bool last = true;
            for (int p = 0; p < c->nranks; ++p)
                if (c->shared->ranks[p].state.load() != 2) last = false;
            if (last) shm_unlink(c->shmName.c_str());
        }
        munmap(c->shared, sizeof(Shared));
        c->shared = nullptr;
    }
    arenaGive(c->device, c->arena);
    c->arena = nullptr;
}

ncclResult_t initRank(ncclComm_t* out, int nranks, const ncclUniqueId& uid, int rank) {
    if (!out || nranks < 1 || rank < 0 || rank >= nranks) return ncclInvalidArgument;
    if (nranks > kMaxRanks) return ncclInvalidArgument;
    IdPayload id;
    std::memcpy(&id, uid.internal, sizeof id);
    if (id.magic != kMagic) return ncclInvalidArgument;
    if (cudaFree(nullptr) != cudaSuccess) return ncclUnhandledCudaError;
    auto* c = new ncclComm;
    c->rank = rank, c->nranks = nranks;
    c->idToken[0] = id.token[0], c->idToken[1] = id.token[1];
    cudaGetDevice(&c->device);
    c->shmName = shmNameOf(id);
    // Any failure from here on gives back what was taken; once this rank's slot is published it is also marked as left, so
    // that the peers' waits end with an error at once instead of running into their timeout.
    const auto giveUp = [&](ncclResult_t r, const char* what, bool published) {
        if (what) fail(nullptr, r, what);
        if (published && c->shared) c->shared->abort.store(1);
        release(c, published);
        delete c;
        return r;
    };
    const int fd = shm_open(c->shmName.c_str(), O_CREAT | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, sizeof(Shared)) != 0) {
        if (fd >= 0) close(fd);
        return giveUp(ncclSystemError, "shm_open failed", false);
    }
    void* mem = mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);  // a new object reads as zeros
    close(fd);
    if (mem == MAP_FAILED) return giveUp(ncclSystemError, "mmap failed", false);
    c->shared = static_cast<Shared*>(mem);
    RankSlot& slot = c->shared->ranks[rank];
    c->arena = arenaTake(c->device, slot.arenaPost);
    if (!c->arena) return giveUp(ncclUnhandledCudaError, "could not allocate or export the flag arena", false);
    slot.pid = int(getpid());
    cudaDeviceGetPCIBusId(slot.busId, sizeof slot.busId, c->device);
    slot.arenaRaw = reinterpret_cast<uint64_t>(c->arena);
    slot.state.store(1, std::memory_order_release);
    const ncclResult_t r = hostWait(c, [&] {
        for (int p = 0; p < nranks; ++p)
            if (c->shared->ranks[p].state.load(std::memory_order_acquire) == 0) return false;
        return true;
    }, "every rank to join the communicator");
    if (r != ncclSuccess) return giveUp(r, nullptr, true);
    for (int p = 0; p < nranks; ++p) {
        const RankSlot& s = c->shared->ranks[p];
        c->samePid[p] = s.pid == slot.pid;
        for (int q = 0; q < p; ++q)
            if (!std::strcmp(c->shared->ranks[q].busId, s.busId)) c->hostSync = true;
        if (p == rank) continue;
        if (c->samePid[p]) {
            c->peerArena[p] = reinterpret_cast<Arena*>(s.arenaRaw);
            int peerDev = -1;
            cudaDeviceGetByPCIBusId(&peerDev, s.busId);
            if (peerDev >= 0 && peerDev != c->device && cudaDeviceEnablePeerAccess(peerDev, 0) != cudaSuccess) cudaGetLastError();
        } else {
            void* base = ipcAcquire(s.pid, s.arenaPost.base, s.arenaPost.handle, c->peerArenaGeneration[p]);
            if (!base) return giveUp(ncclUnhandledCudaError, "cudaIpcOpenMemHandle failed for a peer's flag arena (no peer access between the GPUs?)", true);
            c->peerArenaBase[p] = s.arenaPost.base;
            c->peerArena[p] = reinterpret_cast<Arena*>(static_cast<char*>(base) + s.arenaPost.offset);
        }
    }
    *out = c;
    return ncclSuccess;
}

void destroy(ncclComm* c) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    release(c, true);
    cudaSetDevice(prev);
    delete c;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

ncclResult_t ncclGetVersion(int* version) {
    if (!version) return ncclInvalidArgument;
    *version = NCCL_VERSION_CODE;
    return ncclSuccess;
}

ncclResult_t ncclGetUniqueId(ncclUniqueId* uniqueId) {
    if (!uniqueId) return ncclInvalidArgument;
    std::memset(uniqueId, 0, sizeof *uniqueId);
    std::random_device rd;
    IdPayload id{kMagic, 0, {(uint64_t(rd()) << 32) | rd(), (uint64_t(rd()) << 32) ^ uint64_t(getpid()) ^ uint64_t(std::chrono::steady_clock::now().time_since_epoch().count())}};
    std::memcpy(uniqueId->internal, &id, sizeof id);
    return ncclSuccess;
}

ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank) { return initRank(comm, nranks, commId, rank); }
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank, ncclConfig_t*) {
    return initRank(comm, nranks, commId, rank);
}

// One communicator per listed device, all in this process (nccl.cpp:528-543).
ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
    if (!comms || ndev < 1 || ndev > kMaxRanks) return ncclInvalidArgument;
    ncclUniqueId id;
    ncclGetUniqueId(&id);
    int prev = 0;
    cudaGetDevice(&prev);
    std::vector<ncclResult_t> results(ndev, ncclSuccess);
    std::vector<std::thread> threads;
    for (int r = 0; r < ndev; ++r)
        threads.emplace_back([&, r] {
            if (cudaSetDevice(devlist ? devlist[r] : r) != cudaSuccess) {
                results[r] = ncclInvalidArgument;
                return;
            }
            results[r] = initRank(&comms[r], ndev, id, r);
        });
    for (auto& t : threads) t.join();
    cudaSetDevice(prev);
    for (ncclResult_t r : results)
        if (r != ncclSuccess) return r;
    return ncclSuccess;
}

ncclResult_t ncclCommFinalize(ncclComm_t comm) { return comm ? ncclSuccess : ncclInvalidArgument; }

ncclResult_t ncclCommDestroy(ncclComm_t comm) {
    if (!comm) return ncclSuccess;
    destroy(comm);
    return ncclSuccess;
}

ncclResult_t ncclCommAbort(ncclComm_t comm) {
    if (!comm) return ncclInvalidArgument;
    comm->aborted.store(true);
    if (comm->shared) comm->shared->abort.store(1);
    return ncclSuccess;
}

const char* ncclGetErrorString(ncclResult_t result) {
    switch (result) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error";
    case ncclSystemError: return "unhandled system error";
    case ncclInternalError: return "internal error";
    case ncclInvalidArgument: return "invalid argument";
    case ncclInvalidUsage: return "invalid usage";
    case ncclRemoteError: return "remote process exited or there was a network error";
    case ncclInProgress: return "NCCL operation in progress";
    default: return "unknown result code";
    }
}

const char* ncclGetLastError(ncclComm_t comm) { return comm ? comm->lastError.c_str() : ""; }

// Reads the device status word (a blocking copy): non-zero means a device-side barrier gave up on a peer.
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError) {
    if (!comm || !asyncError) return ncclInvalidArgument;
    unsigned status = 0;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(comm->device);
    const cudaError_t e = cudaMemcpy(&status, &comm->arena->status, sizeof status, cudaMemcpyDeviceToHost);
    cudaSetDevice(prev);
    *asyncError = e != cudaSuccess ? ncclUnhandledCudaError : status || comm->aborted.load() ? ncclRemoteError : ncclSuccess;
    return ncclSuccess;
}

ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) {
    if (!comm || !count) return ncclInvalidArgument;
    *count = comm->nranks;
    return ncclSuccess;
}
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device) {
    if (!comm || !device) return ncclInvalidArgument;
    *device = comm->device;
    return ncclSuccess;
}
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) {
    if (!comm || !rank) return ncclInvalidArgument;
    *rank = comm->rank;
    return ncclSuccess;
}
ncclResult_t ncclCommRegister(const ncclComm_t comm, void* buff, size_t, void** handle) {
    if (!comm || !handle) return ncclInvalidArgument;
    *handle = buff;  // every cudaMalloc buffer is reachable already; nothing to prepare
    return ncclSuccess;
}
ncclResult_t ncclCommDeregister(const ncclComm_t comm, void*) { return comm ? ncclSuccess : ncclInvalidArgument; }
ncclResult_t ncclMemAlloc(void** ptr, size_t size) {
    if (!ptr) return ncclInvalidArgument;
    return cudaMalloc(ptr, size) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
ncclResult_t ncclMemFree(void* ptr) { return cudaFree(ptr) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError; }

ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kAllGather, sendbuff, recvbuff, sendcount, datatype, ncclSum, 0, stream});
}
ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kBroadcast, sendbuff, recvbuff, count, datatype, ncclSum, root, stream});
}
ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kBroadcast, buff, buff, count, datatype, ncclSum, root, stream});
}
ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kAllReduce, sendbuff, recvbuff, count, datatype, op, 0, stream});
}
ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kReduceScatter, sendbuff, recvbuff, recvcount, datatype, op, 0, stream});
}
ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kReduce, sendbuff, recvbuff, count, datatype, op, root, stream});
}
ncclResult_t ncclGather(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kGather, sendbuff, recvbuff, count, datatype, ncclSum, root, stream});
}
ncclResult_t ncclAlltoAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kAllToAll, sendbuff, recvbuff, count, datatype, ncclSum, 0, stream});
}

// Point to point (nccl.cpp:706-715): the n-th send from a rank to a peer matches that peer's n-th receive from the rank.
ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
    Op op{comm, kSend, sendbuff, nullptr, count, datatype, ncclSum, 0, stream};
    op.peer = peer;
    return submit(op);
}
ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
    Op op{comm, kRecv, nullptr, recvbuff, count, datatype, ncclSum, 0, stream};
    op.peer = peer;
    return submit(op);
}

// A sum whose contributions are multiplied by a per-rank scalar first (nccl.cpp:650-666). A scalar in host memory is read
// now; one in device memory is read each time a collective with this operator is issued.
ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype, ncclScalarResidence_t residence, ncclComm_t comm) {
    if (!op || !scalar || !comm || typeSize(datatype) == 0 || datatype == ncclFloat8e4m3 || datatype == ncclFloat8e5m2) return ncclInvalidArgument;
    for (int i = 0; i < kMaxCustomOps; ++i) {
        ncclComm::CustomOp& slot = comm->customOps[i];
        if (slot.live) continue;
        slot.live = true, slot.type = datatype;
        if (residence == ncclScalarHostImmediate) slot.factor = scalarValue(scalar, datatype), slot.devicePointer = nullptr;
        else slot.factor = 1.0, slot.devicePointer = scalar;
        *op = ncclRedOp_t(int(ncclNumOps) + i);
        return ncclSuccess;
    }
    return fail(comm, ncclInvalidUsage, "too many reduction operators alive on this communicator");
}

ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm) {
    const int index = int(op) - int(ncclNumOps);
    if (!comm || index < 0 || index >= kMaxCustomOps || !comm->customOps[index].live) return ncclInvalidArgument;
    comm->customOps[index].live = false;
    return ncclSuccess;
}

// Ranks that pass the same color form a new communicator, ordered by (key, rank here); NCCL_SPLIT_NOCOLOR leaves a rank
// without one (nccl.cpp:561-591). Collective over `comm` and blocking on the host: the (color, key) pairs travel through the
// shared-memory object, and the members of a color derive their new communicator's id from this communicator's.
ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t*) {
    if (!comm || !newcomm) return ncclInvalidArgument;
    *newcomm = nullptr;
    const uint64_t seq = ++comm->splitCount;
    RankSlot& mine = comm->shared->ranks[comm->rank];
    // nobody may still be reading the previous split's pairs
    ncclResult_t r = hostWait(comm, [&] {
        for (int p = 0; p < comm->nranks; ++p)
            if (comm->shared->ranks[p].splitRead.load(std::memory_order_acquire) < seq - 1) return false;
        return true;
    }, "the other ranks to finish the previous split");
    if (r != ncclSuccess) return r;
    mine.splitColor = color, mine.splitKey = key;
    mine.splitSeq.store(seq, std::memory_order_release);
    r = hostWait(comm, [&] {
        for (int p = 0; p < comm->nranks; ++p)
            if (comm->shared->ranks[p].splitSeq.load(std::memory_order_acquire) < seq) return false;
        return true;
    }, "the other ranks to enter ncclCommSplit");
    if (r != ncclSuccess) return r;
    int members = 0, myRank = 0;
    for (int p = 0; p < comm->nranks; ++p) {
        const RankSlot& s = comm->shared->ranks[p];
        if (s.splitColor != color) continue;
        ++members;
        if (s.splitKey < key || (s.splitKey == key && p < comm->rank)) ++myRank;
    }
    mine.splitRead.store(seq, std::memory_order_release);
    if (color == NCCL_SPLIT_NOCOLOR) return ncclSuccess;
    if (color < 0) return fail(comm, ncclInvalidArgument, "a color is not negative");
    ncclUniqueId id;
    std::memset(&id, 0, sizeof id);
    // the same words on every member, different for every (parent, split number, color)
    IdPayload payload{kMagic, 0, {comm->idToken[0] * 0x9E3779B97F4A7C15ull + seq * 0xBF58476D1CE4E5B9ull + uint64_t(color) + 1,
                                  comm->idToken[1] ^ (seq << 32) ^ (uint64_t(color) * 0x94D049BB133111EBull)}};
    std::memcpy(id.internal, &payload, sizeof payload);
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(comm->device);
    r = initRank(newcomm, members, id, myRank);
    cudaSetDevice(prev);
    return r;
}

// Diagnostic: runs this communicator's device-side barrier against a peer that does not exist (a flag word nobody writes),
// so the bounded wait runs out: the kernel returns after the device wait limit (VKZB_NCCL_DEVICE_WAIT_MS) and
// ncclCommGetAsyncError reports ncclRemoteError. Nothing faults and the context stays usable; lets an installation check
// that a lost peer is noticed. The communicator should be destroyed afterwards (its status word stays set).
ncclResult_t vkzbNcclSelfTestLostPeer(ncclComm_t comm, cudaStream_t stream) {
    if (!comm) return ncclInvalidArgument;
    if (comm->nranks > kMaxRanks - 2) return ncclInvalidUsage;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(comm->device);
    // As "rank 0 of 2" on the two highest flag words of this rank's own arena, which no real peer uses below 15 ranks: the
    // kernel stores its arrival into the first and waits for the second, which nobody ever writes.
    FlagTable t{};
    unsigned long long* spare = &comm->arena->flags[kMaxRanks - 2];
    t.peer[1] = spare;
    barrierKernel<<<1, 32, 0, stream>>>(t, spare, &comm->arena->status, 0, 2, 1ull, deviceWaitNs());
    const cudaError_t e = cudaGetLastError();
    cudaSetDevice(prev);
    return e == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

ncclResult_t ncclGroupStart(void) {
    ++t_groupDepth;
    return ncclSuccess;
}

ncclResult_t ncclGroupEnd(void) {
    if (t_groupDepth <= 0) return ncclInvalidUsage;
    if (--t_groupDepth > 0) return ncclSuccess;
    std::vector<Op> ops;
    ops.swap(t_queue);
    if (ops.empty()) return ncclSuccess;
    int prev = 0;
    cudaGetDevice(&prev);
    const ncclResult_t r = execute(ops);
    cudaSetDevice(prev);
    return r;
}


// ---- extensions (include/vkzb_nccl.h): what a kernel that writes its results straight into its peers needs ----

// Collective and blocking on the host only: every rank hands in one cudaMalloc'ed buffer and gets back, for each rank, an
// address through which this process reaches that rank's buffer (its own for its own rank).
ncclResult_t vkzbNcclExchangeBuffer(ncclComm_t comm, void* buffer, void** peers) {
    if (!comm || !buffer || !peers) return ncclInvalidArgument;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(comm->device);
    ncclResult_t result = ncclSuccess;
    const uint64_t seq = ++comm->opSeq;
    peers[comm->rank] = buffer;
    if (comm->nranks > 1) {
        RankSlot& slot = comm->shared->ranks[comm->rank];
        OpPost& post = slot.posts[seq % kPostRing];
        BufferPost none{};
        post.recv = none;
        if (!describeBuffer(buffer, post.send)) result = fail(comm, ncclInvalidArgument, "the buffer is not device memory that can be shared (cudaMalloc memory is)");
        slot.postSeq.store(seq, std::memory_order_release);  // published even on failure, so the peers do not wait for it
        if (result == ncclSuccess)
            result = hostWait(comm, [&] {
                for (int p = 0; p < comm->nranks; ++p)
                    if (comm->shared->ranks[p].postSeq.load(std::memory_order_acquire) < seq) return false;
                return true;
            }, "the other ranks to hand in their buffer");
        for (int p = 0; result == ncclSuccess && p < comm->nranks; ++p) {
            if (p == comm->rank) continue;
            peers[p] = mapPeerBuffer(comm, p, comm->shared->ranks[p].posts[seq % kPostRing].send);
            if (!peers[p]) result = fail(comm, ncclUnhandledCudaError, "could not map a peer's buffer (cudaIpcOpenMemHandle)");
        }
    }
    cudaSetDevice(prev);
    return result;
}

// A barrier across the ranks, asynchronous on `stream` (on the host where ranks share a GPU): work enqueued after it on any
// rank starts only when every rank's stream has reached it.
ncclResult_t vkzbNcclBarrier(ncclComm_t comm, cudaStream_t stream) {
    return submit({comm, kBarrierOnly, nullptr, nullptr, 0, ncclInt8, ncclSum, 0, stream});
}

// Not served yet (include/vkzb_nccl.h lists them): parameterless like the reference's stubs, so any signature binds.
#define VKZB_NCCL_STUB(name) \
    ncclResult_t name() { return ncclInvalidUsage; }
VKZB_NCCL_STUB(ncclCommInitRankScalable)
VKZB_NCCL_STUB(ncclGroupSimulateEnd)
VKZB_NCCL_STUB(ncclCommGetUniqueId)
VKZB_NCCL_STUB(ncclCommGrow)
VKZB_NCCL_STUB(ncclCommMemStats)
VKZB_NCCL_STUB(ncclCommResume)
VKZB_NCCL_STUB(ncclCommRevoke)
VKZB_NCCL_STUB(ncclCommShrink)
VKZB_NCCL_STUB(ncclCommSuspend)
VKZB_NCCL_STUB(ncclCommWindowDeregister)
VKZB_NCCL_STUB(ncclCommWindowRegister)
VKZB_NCCL_STUB(ncclDevCommCreate)
VKZB_NCCL_STUB(ncclDevCommDestroy)
VKZB_NCCL_STUB(ncclGetLsaMultimemDevicePointer)
VKZB_NCCL_STUB(ncclGetPeerDevicePointer)
VKZB_NCCL_STUB(ncclPutSignal)
VKZB_NCCL_STUB(ncclSignal)
VKZB_NCCL_STUB(ncclWaitSignal)
VKZB_NCCL_STUB(ncclWinGetUserPtr)

}  // extern "C"
#pragma GCC visibility pop
