#include "gpu/symm_heap.hpp"

#include <fcntl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/syscall.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <thread>

#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/device/layout.hpp"

namespace cclx {
namespace gpu {

static size_t round_up(size_t v, size_t a) {
    return (v + a - 1) / a * a;
}

heap_regions plan_regions(int world, size_t heap_bytes, size_t staging_bytes, size_t granularity) {
    heap_regions r;
    size_t off = 0;
    r.flags_off = off;
    off += round_up((size_t)dev::MAX_BLOCKS * dev::MAX_RANKS * sizeof(uint32_t), 4096);
    r.p2p_flags_off = off;
    off += round_up((size_t)dev::P2P_PAGE_WORDS * sizeof(uint32_t), 4096);
    r.aux_flags_off = off;
    r.aux_flags_bytes = 1u << 20;
    off += r.aux_flags_bytes;
    r.p2p_slot_bytes = dev::P2P_SLOT_BYTES;
    r.p2p_data_off = off;
    off += (size_t)world * r.p2p_slot_bytes;
    off = round_up(off, 1u << 20);
    r.staging_off = off;
    r.staging_bytes = round_up(staging_bytes, 4096);
    off += 2 * r.staging_bytes;
    off = round_up(off, 1u << 20);
    r.user_off = off;
    // the requested size covers flags, staging and the user part; the point-to-point slots come on top
    r.total = round_up(std::max(off + (1u << 20), heap_bytes + (size_t)world * r.p2p_slot_bytes), granularity);
    return r;
}

// ---- fd passing -----------------------------------------------------------------

namespace {

sockaddr_un abstract_addr(const std::string& name, socklen_t& len) {
    sockaddr_un a;
    std::memset(&a, 0, sizeof(a));
    a.sun_family = AF_UNIX;
    // abstract namespace: leading NUL, no file system entry to clean up
    size_t n = std::min(name.size(), sizeof(a.sun_path) - 2);
    std::memcpy(a.sun_path + 1, name.data(), n);
    len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
    return a;
}

bool send_fd(int sock, const sockaddr_un& to, socklen_t tolen, int fd, int src_rank) {
    msghdr msg;
    std::memset(&msg, 0, sizeof(msg));
    char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    iovec iov;
    iov.iov_base = &src_rank;
    iov.iov_len = sizeof(src_rank);
    msg.msg_name = const_cast<sockaddr_un*>(&to);
    msg.msg_namelen = tolen;
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(cm), &fd, sizeof(int));
    ssize_t n = sendmsg(sock, &msg, MSG_DONTWAIT);
    if (n < 0) {
        if (errno == EAGAIN || errno == EWOULDBLOCK || errno == ENOBUFS || errno == ECONNREFUSED ||
            errno == ENOENT)
            return false;
        CCL_THROW("sendmsg(SCM_RIGHTS) failed: ", std::strerror(errno));
    }
    return true;
}

bool recv_fd(int sock, int& fd, int& src_rank) {
    msghdr msg;
    std::memset(&msg, 0, sizeof(msg));
    char ctrl[CMSG_SPACE(sizeof(int))];
    iovec iov;
    iov.iov_base = &src_rank;
    iov.iov_len = sizeof(src_rank);
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n = recvmsg(sock, &msg, MSG_DONTWAIT);
    if (n < 0) {
        if (errno == EAGAIN || errno == EWOULDBLOCK)
            return false;
        CCL_THROW("recvmsg failed: ", std::strerror(errno));
    }
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    CCL_THROW_IF_NOT(cm && cm->cmsg_type == SCM_RIGHTS, "message without a descriptor");
    std::memcpy(&fd, CMSG_DATA(cm), sizeof(int));
    return true;
}

// generic: rank r sends `give[p]` (or -1 = nothing) to p and expects a fd from
// every p with expect[p] true.  Returns received fds indexed by source.
std::vector<int> fd_rounds(bootstrap_if& bs, const std::vector<int>& give, const std::vector<bool>& expect,
                           const std::string& tag) {
    const int W = bs.size(), me = bs.rank();
    const std::string prefix = "cclx-" + bs.job_id() + "-" + tag + "-";
    int sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    CCL_THROW_IF_NOT(sock >= 0, "socket(AF_UNIX) failed: ", std::strerror(errno));
    socklen_t mylen;
    sockaddr_un mine = abstract_addr(prefix + std::to_string(me), mylen);
    CCL_THROW_IF_NOT(bind(sock, (sockaddr*)&mine, mylen) == 0, "bind failed: ", std::strerror(errno));
    bs.barrier(); // every socket is bound

    std::vector<int> got(W, -1);
    std::vector<bool> sent(W, false);
    int to_send = 0, to_recv = 0;
    for (int p = 0; p < W; p++) {
        if (p != me && give[p] >= 0)
            to_send++;
        if (p != me && expect[p])
            to_recv++;
    }
    auto t0 = std::chrono::steady_clock::now();
    while (to_send > 0 || to_recv > 0) {
        bool progress = false;
        for (int p = 0; p < W && to_send > 0; p++) {
            if (p == me || give[p] < 0 || sent[p])
                continue;
            socklen_t l;
            sockaddr_un a = abstract_addr(prefix + std::to_string(p), l);
            if (send_fd(sock, a, l, give[p], me)) {
                sent[p] = true;
                to_send--;
                progress = true;
            }
        }
        while (to_recv > 0) {
            int fd = -1, src = -1;
            if (!recv_fd(sock, fd, src))
                break;
            CCL_THROW_IF_NOT(src >= 0 && src < W && got[src] < 0, "unexpected descriptor from rank ", src);
            got[src] = fd;
            to_recv--;
            progress = true;
        }
        if (!progress) {
            std::this_thread::sleep_for(std::chrono::microseconds(200));
            auto dt = std::chrono::steady_clock::now() - t0;
            CCL_THROW_IF_NOT(dt < std::chrono::seconds(env_data::get().kvs_connection_timeout_sec),
                             "timed out exchanging memory handles");
        }
    }
    bs.barrier(); // nobody sends to a closed socket
    close(sock);
    return got;
}

int sys_pidfd_open(pid_t pid) {
    return (int)syscall(434 /* pidfd_open */, pid, 0);
}
int sys_pidfd_getfd(int pidfd, int fd) {
    return (int)syscall(438 /* pidfd_getfd */, pidfd, fd, 0);
}

} // namespace

std::vector<int> exchange_fds_sockets(bootstrap_if& bs, int my_fd, const std::string& tag) {
    const int W = bs.size();
    std::vector<int> give(W, my_fd);
    std::vector<bool> expect(W, true);
    return fd_rounds(bs, give, expect, tag);
}

std::vector<int> exchange_fds_pidfd(bootstrap_if& bs, int my_fd) {
    const int W = bs.size(), me = bs.rank();
    struct rec {
        int pid;
        int fd;
    } mine{ (int)getpid(), my_fd };
    std::vector<rec> all(W);
    bs.allgather(&mine, all.data(), sizeof(rec));
    std::vector<int> got(W, -1);
    for (int p = 0; p < W; p++) {
        if (p == me)
            continue;
        int pidfd = sys_pidfd_open(all[p].pid);
        CCL_THROW_IF_NOT(pidfd >= 0, "pidfd_open(", all[p].pid, ") failed: ", std::strerror(errno));
        got[p] = sys_pidfd_getfd(pidfd, all[p].fd);
        int e = errno;
        close(pidfd);
        CCL_THROW_IF_NOT(got[p] >= 0, "pidfd_getfd failed: ", std::strerror(e),
                         " (needs ptrace permission; use CCL_CUDA_IPC_EXCHANGE=sockets)");
    }
    bs.barrier(); // owners keep their descriptors open until everybody duplicated them
    return got;
}

static int bcast_fd(bootstrap_if& bs, int root, int fd, ipc_exchange_t mode, const std::string& tag) {
    const int W = bs.size(), me = bs.rank();
    if (mode == ipc_exchange_t::pidfd) {
        struct rec {
            int pid;
            int fd;
        } mine{ (int)getpid(), fd };
        std::vector<rec> all(W);
        bs.allgather(&mine, all.data(), sizeof(rec));
        int out = fd;
        if (me != root) {
            int pidfd = sys_pidfd_open(all[root].pid);
            CCL_THROW_IF_NOT(pidfd >= 0, "pidfd_open failed: ", std::strerror(errno));
            out = sys_pidfd_getfd(pidfd, all[root].fd);
            close(pidfd);
            CCL_THROW_IF_NOT(out >= 0, "pidfd_getfd failed: ", std::strerror(errno));
        }
        bs.barrier();
        return out;
    }
    std::vector<int> give(W, -1);
    std::vector<bool> expect(W, false);
    if (me == root)
        std::fill(give.begin(), give.end(), fd);
    else
        expect[root] = true;
    std::vector<int> got = fd_rounds(bs, give, expect, tag);
    return me == root ? fd : got[root];
}

// ---- heap ---------------------------------------------------------------------

symm_heap::~symm_heap() {
    try {
        destroy();
    }
    catch (...) {
    }
}

void symm_heap::create_emulated(int world, size_t heap_bytes, size_t staging_bytes) {
    CCL_THROW_IF_NOT(world >= 1 && world <= dev::MAX_RANKS, "emulated world out of range");
    emulated_ = true;
    world_ = world;
    rank_ = 0;
    regions_ = plan_regions(world, heap_bytes, staging_bytes, 1u << 20);
    bases_.assign(world, nullptr);
    for (int r = 0; r < world; r++) {
        void* p = nullptr;
        CUDA_CHECK(cudaMalloc(&p, regions_.total));
        CUDA_CHECK(cudaMemset(p, 0, regions_.user_off));
        bases_[r] = (char*)p;
    }
    free_.clear();
    used_.clear();
    free_[regions_.user_off] = regions_.total - regions_.user_off;
}

void symm_heap::create(bootstrap_if& bs, size_t heap_bytes, size_t staging_bytes, ipc_exchange_t mode, int nvls) {
    const driver_api& d = driver();
    CCL_THROW_IF_NOT(d.loaded, "CUDA driver not available: ", d.error);
    rank_ = bs.rank();
    world_ = bs.size();
    CCL_THROW_IF_NOT(world_ <= dev::MAX_RANKS, "at most ", dev::MAX_RANKS, " ranks per node communicator");
    emulated_ = false;
    CUDA_CHECK(cudaGetDevice(&device_));
    CUDA_CHECK(cudaFree(0)); // make sure the primary context exists
    CUdevice cudev;
    CU_CHECK(d.DeviceGet(&cudev, device_));

    int fabric_ok = 0, mc_ok = 0;
    d.DeviceGetAttribute(&fabric_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED, cudev);
    d.DeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev);
    if (mode == ipc_exchange_t::fabric && !fabric_ok) {
        LOG_WARN("fabric handles not supported on this device, using sockets");
        mode = ipc_exchange_t::sockets;
    }
    if (mode == ipc_exchange_t::cudaipc)
        mode = ipc_exchange_t::sockets; // legacy cudaIpc handles cannot be bound to NVLS; same capability via fd
    const CUmemAllocationHandleType htype =
        mode == ipc_exchange_t::fabric ? CU_MEM_HANDLE_TYPE_FABRIC : CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    bool want_mc = (nvls != 0) && mc_ok && d.MulticastCreate && world_ > 1;
    if (nvls == 1 && !want_mc)
        LOG_WARN("CCL_CUDA_NVLS=1 but multicast is not supported here");
    // all ranks must agree
    {
        int mine = want_mc ? 1 : 0;
        std::vector<int> all(world_);
        bs.allgather(&mine, all.data(), sizeof(int));
        for (int v : all)
            want_mc = want_mc && v;
    }

    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device_;
    prop.requestedHandleTypes = htype;
    size_t gran = 0;
    CU_CHECK(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    CUmulticastObjectProp mprop;
    std::memset(&mprop, 0, sizeof(mprop));
    if (want_mc) {
        mprop.numDevices = (unsigned)world_;
        mprop.handleTypes = htype;
        mprop.flags = 0;
        mprop.size = gran; // provisional, for the granularity query
        size_t mgran = 0;
        CU_CHECK(d.MulticastGetGranularity(&mgran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED));
        gran = std::max(gran, mgran);
    }
    regions_ = plan_regions(world_, heap_bytes, staging_bytes, gran);
    const size_t total = regions_.total;

    CUmemGenericAllocationHandle myh;
    CU_CHECK(d.MemCreate(&myh, total, &prop, 0));
    handles_.assign(world_, 0);
    handles_[rank_] = myh;

    // ---- exchange handles
    if (htype == CU_MEM_HANDLE_TYPE_FABRIC) {
        CUmemFabricHandle fh;
        CU_CHECK(d.MemExportToShareableHandle(&fh, myh, htype, 0));
        std::vector<CUmemFabricHandle> all(world_);
        bs.allgather(&fh, all.data(), sizeof(fh));
        for (int p = 0; p < world_; p++) {
            if (p == rank_)
                continue;
            CUmemGenericAllocationHandle h;
            CU_CHECK(d.MemImportFromShareableHandle(&h, &all[p], htype));
            handles_[p] = h;
        }
    }
    else {
        int myfd = -1;
        CU_CHECK(d.MemExportToShareableHandle(&myfd, myh, htype, 0));
        std::vector<int> fds = mode == ipc_exchange_t::pidfd ? exchange_fds_pidfd(bs, myfd)
                                                            : exchange_fds_sockets(bs, myfd, "heap");
        for (int p = 0; p < world_; p++) {
            if (p == rank_)
                continue;
            CUmemGenericAllocationHandle h;
            CU_CHECK(d.MemImportFromShareableHandle(&h, (void*)(uintptr_t)fds[p], htype));
            handles_[p] = h;
            close(fds[p]);
        }
        close(myfd);
    }

    // ---- map everything
    CUmemAccessDesc acc;
    std::memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    bases_.assign(world_, nullptr);
    for (int p = 0; p < world_; p++) {
        CUdeviceptr va = 0;
        CU_CHECK(d.MemAddressReserve(&va, total, gran, 0, 0));
        CU_CHECK(d.MemMap(va, total, 0, handles_[p], 0));
        CU_CHECK(d.MemSetAccess(va, total, &acc, 1));
        bases_[p] = (char*)va;
    }
    mapped_bytes_ = total;
    CUDA_CHECK(cudaMemset(bases_[rank_], 0, regions_.user_off));
    CUDA_CHECK(cudaDeviceSynchronize());

    // ---- NVLS multicast window
    if (want_mc) {
        mprop.size = total;
        CUmemGenericAllocationHandle mch = 0;
        bool ok = true;
        if (htype == CU_MEM_HANDLE_TYPE_FABRIC) {
            CUmemFabricHandle fh;
            std::memset(&fh, 0, sizeof(fh));
            if (rank_ == 0) {
                CU_CHECK(d.MulticastCreate(&mch, &mprop));
                CU_CHECK(d.MemExportToShareableHandle(&fh, mch, htype, 0));
            }
            std::vector<CUmemFabricHandle> all(world_);
            bs.allgather(&fh, all.data(), sizeof(fh));
            if (rank_ != 0)
                CU_CHECK(d.MemImportFromShareableHandle(&mch, &all[0], htype));
        }
        else {
            int fd = -1;
            int created = 1;
            if (rank_ == 0) {
                CUresult r = d.MulticastCreate(&mch, &mprop);
                if (r != CUDA_SUCCESS) {
                    LOG_WARN("cuMulticastCreate failed (", cu_error_string(r), "), NVLS disabled");
                    created = 0;
                }
                else
                    CU_CHECK(d.MemExportToShareableHandle(&fd, mch, htype, 0));
            }
            std::vector<int> flags(world_);
            bs.allgather(&created, flags.data(), sizeof(int));
            ok = flags[0] != 0;
            if (ok) {
                int got = bcast_fd(bs, 0, fd, mode, "mc");
                if (rank_ != 0) {
                    CU_CHECK(d.MemImportFromShareableHandle(&mch, (void*)(uintptr_t)got, htype));
                    close(got);
                }
                else
                    close(fd);
            }
        }
        if (ok) {
            CU_CHECK(d.MulticastAddDevice(mch, cudev));
            bs.barrier(); // every device added before anyone binds
            CU_CHECK(d.MulticastBindMem(mch, 0, myh, 0, total, 0));
            mc_bound_ = true;
            bs.barrier();
            CUdeviceptr va = 0;
            CU_CHECK(d.MemAddressReserve(&va, total, gran, 0, 0));
            CU_CHECK(d.MemMap(va, total, 0, mch, 0));
            CU_CHECK(d.MemSetAccess(va, total, &acc, 1));
            mc_base_ = (char*)va;
            mc_handle_ = mch;
            LOG_INFO("NVLS multicast window mapped, ", total >> 20, " MiB");
        }
    }
    bs.barrier();
    free_.clear();
    used_.clear();
    free_[regions_.user_off] = regions_.total - regions_.user_off;
    LOG_INFO("symmetric heap ready: ", total >> 20, " MiB per rank, staging 2 x ", regions_.staging_bytes >> 20,
             " MiB, nvls=", has_multicast());
}

void symm_heap::destroy() {
    if (bases_.empty())
        return;
    if (emulated_) {
        for (char* p : bases_)
            if (p)
                cudaFree(p);
        bases_.clear();
        return;
    }
    const driver_api& d = driver();
    cudaDeviceSynchronize();
    if (mc_base_) {
        d.MemUnmap((CUdeviceptr)mc_base_, mapped_bytes_);
        d.MemAddressFree((CUdeviceptr)mc_base_, mapped_bytes_);
        mc_base_ = nullptr;
    }
    if (mc_handle_) {
        if (mc_bound_) {
            CUdevice cudev;
            if (d.DeviceGet(&cudev, device_) == CUDA_SUCCESS)
                d.MulticastUnbind((CUmemGenericAllocationHandle)mc_handle_, cudev, 0, mapped_bytes_);
            mc_bound_ = false;
        }
        d.MemRelease((CUmemGenericAllocationHandle)mc_handle_);
        mc_handle_ = 0;
    }
    for (int p = 0; p < world_; p++) {
        if (bases_[p]) {
            d.MemUnmap((CUdeviceptr)bases_[p], mapped_bytes_);
            d.MemAddressFree((CUdeviceptr)bases_[p], mapped_bytes_);
        }
        if (handles_[p])
            d.MemRelease((CUmemGenericAllocationHandle)handles_[p]);
    }
    bases_.clear();
    handles_.clear();
}

size_t symm_heap::alloc(size_t bytes) {
    bytes = round_up(std::max<size_t>(bytes, 1), 256);
    for (auto it = free_.begin(); it != free_.end(); ++it) {
        if (it->second >= bytes) {
            size_t off = it->first, len = it->second;
            free_.erase(it);
            if (len > bytes)
                free_[off + bytes] = len - bytes;
            used_[off] = bytes;
            return off;
        }
    }
    CCL_THROW("symmetric heap exhausted: need ", bytes, " bytes, free ", user_bytes_free(),
              "; raise CCL_CUDA_SYMM_HEAP_SIZE");
}

void symm_heap::free(size_t off) {
    auto it = used_.find(off);
    CCL_THROW_IF_NOT(it != used_.end(), "free of unknown symmetric offset ", off);
    size_t len = it->second;
    used_.erase(it);
    auto ins = free_.emplace(off, len).first;
    // merge with next
    auto nx = std::next(ins);
    if (nx != free_.end() && ins->first + ins->second == nx->first) {
        ins->second += nx->second;
        free_.erase(nx);
    }
    if (ins != free_.begin()) {
        auto pv = std::prev(ins);
        if (pv->first + pv->second == ins->first) {
            pv->second += ins->second;
            free_.erase(ins);
        }
    }
}

size_t symm_heap::user_bytes_free() const {
    size_t s = 0;
    for (auto& kv : free_)
        s += kv.second;
    return s;
}

size_t symm_heap::offset_of(const void* p, int owner_rank) const {
    if (owner_rank < 0 || owner_rank >= (int)bases_.size() || !bases_[owner_rank])
        return (size_t)-1;
    const char* b = bases_[owner_rank];
    const char* q = (const char*)p;
    if (q >= b + regions_.user_off && q < b + regions_.total)
        return (size_t)(q - b);
    return (size_t)-1;
}

} // namespace gpu
} // namespace cclx
