// TCP mesh transport: one non-blocking socket per (endpoint, peer), tag matching
// with posted / unexpected queues, progress driven by poll().
//
// Stands where the reference has atl_ofi with the tcp provider
// (src/atl/ofi/atl_ofi.cpp:30-1196: tagged send/recv, per-worker endpoints,
// address table exchanged through PMI), written directly on sockets: the
// address table is the list of "<ip>:<port>" strings published in the KVS, the
// higher rank of a pair dials the lower one, and a 16-byte header (tag, length)
// frames every message so that a receive posted later still matches.
//
// Pairs of ranks on one host talk through shared memory instead (the reference's
// shm provider, src/atl/ofi/atl_ofi_helper.cpp:1040-1393 picks "shm" beside the
// network provider): every rank owns a POSIX shared-memory segment with one
// single-producer / single-consumer byte ring per (endpoint, sender).  A ring
// carries the same framed byte stream as a socket, so the matching logic is
// shared; only the two functions that move bytes differ.
#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/epoll.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <ctime>
#include <deque>
#include <list>
#include <mutex>
#include <string>

#include "bootstrap/pmi.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "transport/atl.hpp"

namespace cclx {

namespace {

struct wire_header {
    uint64_t tag;
    uint64_t len;
};

struct out_msg {
    wire_header hdr;
    const char* payload;
    size_t sent = 0; // of header + payload
    atl_req* req;
    std::vector<char> owned; // payload kept by the message itself (one-sided writes carried as messages)
    size_t payload_len = 0; // bytes that follow the header on the wire (hdr.len may announce more: rendezvous)
};

// Rendezvous between processes of one host: a long message travels as a descriptor of the sender's
// buffer; the receiver copies it straight into the posted buffer (process_vm_readv: one copy instead of
// one into the ring and one out of it) and acknowledges, which completes the send.  The length field of
// the header carries the flag, the descriptor follows as payload.
constexpr uint64_t RNDV_FLAG = 1ull << 63;
constexpr uint64_t RNDV_ACK_TAG = ~0ull - 1; // payload: the cookie of the descriptor
struct rndv_desc {
    uint64_t addr;
    uint64_t cookie; // the sender's request, echoed in the acknowledgement
    int32_t pid;
    int32_t pad;
};

// tag of a one-sided write that travels as a message: payload = target address, then the data.
// No schedule produces it (communicator id, schedule id and operation id all at their maxima).
constexpr uint64_t RMA_WRITE_TAG = ~0ull;

struct posted_recv {
    uint64_t tag;
    char* buf;
    size_t cap;
    atl_req* req;
};

struct unexpected_msg {
    uint64_t tag;
    std::vector<char> data;
    bool complete = false;
    bool rndv = false; // no data yet: `desc` says where the sender keeps them
    uint64_t rndv_len = 0;
    rndv_desc desc{};
    size_t size() const { return rndv ? (size_t)rndv_len : data.size(); }
};

// single-producer / single-consumer byte ring in shared memory
struct shm_ring {
    alignas(64) std::atomic<uint64_t> head; // bytes written so far (producer)
    alignas(64) std::atomic<uint64_t> tail; // bytes read so far (consumer)
    alignas(64) char data[1];

    static size_t footprint(size_t cap) { return offsetof(shm_ring, data) + cap; }

    size_t write(const void* src, size_t n, size_t cap) {
        const uint64_t h = head.load(std::memory_order_relaxed);
        const uint64_t t = tail.load(std::memory_order_acquire);
        const size_t room = cap - (size_t)(h - t);
        n = std::min(n, room);
        if (n == 0)
            return 0;
        const size_t pos = (size_t)(h & (cap - 1));
        const size_t first = std::min(n, cap - pos);
        std::memcpy(data + pos, src, first);
        std::memcpy(data, (const char*)src + first, n - first);
        head.store(h + n, std::memory_order_release);
        return n;
    }
    size_t read(void* dst, size_t n, size_t cap) {
        const uint64_t t = tail.load(std::memory_order_relaxed);
        const uint64_t h = head.load(std::memory_order_acquire);
        n = std::min(n, (size_t)(h - t));
        if (n == 0)
            return 0;
        const size_t pos = (size_t)(t & (cap - 1));
        const size_t first = std::min(n, cap - pos);
        std::memcpy(dst, data + pos, first);
        std::memcpy((char*)dst + first, data, n - first);
        tail.store(t + n, std::memory_order_release);
        return n;
    }
    bool readable() const {
        return head.load(std::memory_order_acquire) != tail.load(std::memory_order_relaxed);
    }
};

struct peer_state {
    int fd = -1;
    shm_ring* tx = nullptr; // ring in the peer's segment that this rank fills
    shm_ring* rx = nullptr; // ring in this rank's segment that the peer fills
    std::deque<out_msg> outq;
    // incoming
    wire_header in_hdr{};
    size_t hdr_got = 0;
    bool in_body = false;
    char* in_dst = nullptr;
    size_t in_got = 0;
    atl_req* in_req = nullptr; // when receiving straight into a posted buffer
    unexpected_msg* in_unexp = nullptr;
    bool closed = false; // the socket reported end of stream or a reset
    bool dead = false; // the peer is gone: nothing more will arrive, nothing can be delivered
    std::vector<atl_req*> awaiting_ack; // rendezvous sends the peer has not read yet
    size_t body_len = 0; // payload bytes of the message being received
    bool in_ctrl = false; // the payload is a descriptor or an acknowledgement, received into `ctrl`
    char ctrl[sizeof(rndv_desc)];
    std::list<posted_recv> posted;
    std::list<unexpected_msg> unexp;
};

struct endpoint {
    std::vector<peer_state> peers;
    std::vector<int> shm_peers;
    std::mutex mu;
    int epfd = -1;
    uint64_t last_liveness_ns = 0;
    uint64_t liveness_tick = 0;
};

void set_nonblock(int fd) {
    int fl = fcntl(fd, F_GETFL, 0);
    fcntl(fd, F_SETFL, fl | O_NONBLOCK);
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int sz = 4 << 20;
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &sz, sizeof(sz));
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
}

bool write_blocking(int fd, const void* b, size_t n) {
    const char* p = (const char*)b;
    while (n) {
        ssize_t r = ::send(fd, p, n, MSG_NOSIGNAL);
        if (r < 0) {
            if (errno == EINTR)
                continue;
            return false;
        }
        p += r;
        n -= (size_t)r;
    }
    return true;
}
bool read_blocking(int fd, void* b, size_t n) {
    char* p = (char*)b;
    while (n) {
        ssize_t r = ::recv(fd, p, n, 0);
        if (r <= 0) {
            if (r < 0 && errno == EINTR)
                continue;
            return false;
        }
        p += r;
        n -= (size_t)r;
    }
    return true;
}

class tcp_transport : public atl_transport {
public:
    tcp_transport(pmi& pm, int ep_count) : rank_(pm.rank()), size_(pm.size()), eps_(ep_count) {
        const env_data& env = env_data::get();
        // listening socket on the interface the KVS uses
        std::string ip = kvs::choose_local_ip(env.kvs_iface, false);
        if (ip.find(':') != std::string::npos)
            ip = "127.0.0.1";
        int lfd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        CCL_THROW_IF_NOT(lfd >= 0, "socket failed");
        int one = 1;
        setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in a{};
        a.sin_family = AF_INET;
        a.sin_addr.s_addr = htonl(INADDR_ANY);
        a.sin_port = 0;
        CCL_THROW_IF_NOT(::bind(lfd, (sockaddr*)&a, sizeof(a)) == 0, "bind failed: ", std::strerror(errno));
        CCL_THROW_IF_NOT(::listen(lfd, 4096) == 0, "listen failed");
        socklen_t sl = sizeof(a);
        getsockname(lfd, (sockaddr*)&a, &sl);
        char host[256] = { 0 };
        gethostname(host, sizeof(host) - 1);
        struct rec {
            char ip[64];
            int port;
            char host[64];
            int pid;
            uint64_t probe; // address of a word every rank of this host tries to read
        } mine{};
        static const uint64_t probe_word = 0x636d615f70726f62ull;
        mine.pid = (int)getpid();
        mine.probe = (uint64_t)(uintptr_t)&probe_word;
        std::snprintf(mine.ip, sizeof(mine.ip), "%s", ip.c_str());
        mine.port = ntohs(a.sin_port);
        std::snprintf(mine.host, sizeof(mine.host), "%s", host);
        std::vector<rec> table(size_);
        pm.allgather(&mine, table.data(), sizeof(rec));
        same_host_.resize(size_);
        for (int r = 0; r < size_; r++)
            same_host_[r] = std::strncmp(table[r].host, mine.host, sizeof(mine.host)) == 0;
        // can this process read a neighbour's memory?  (ptrace policy and containers may forbid it; the
        // answer is assumed to be the same in both directions between processes of one job on one host)
        // Which same-host peers live in this pid namespace?  Reading a known word out of the peer answers it
        // (a pid alone could belong to an unrelated process of another container).  A verified pid serves the
        // liveness check; cross-memory transfers need every same-host peer verified, and the answer is
        // assumed to be the same in both directions between processes of one job.
        pids_.assign(size_, 0);
        bool all_readable = true;
        for (int r = 0; r < size_; r++) {
            if (r == rank_ || !same_host_[r])
                continue;
            uint64_t got = 0;
            iovec l{ &got, sizeof(got) };
            iovec rm{ (void*)(uintptr_t)table[r].probe, sizeof(got) };
            if (process_vm_readv(table[r].pid, &l, 1, &rm, 1, 0) == (ssize_t)sizeof(got) && got == probe_word)
                pids_[r] = table[r].pid;
            else
                all_readable = false;
        }
        rndv_min_ = (env.atl_cma && all_readable) ? env.atl_cma_threshold : 0;
        if (env.atl_cma && !all_readable) {
            LOG_INFO("process_vm_readv is not permitted between the ranks of this host: long messages go through the rings");
            cma_ok_.store(false, std::memory_order_relaxed);
        }

        for (auto& ep : eps_) {
            ep.peers.resize(size_);
            ep.epfd = epoll_create1(EPOLL_CLOEXEC);
        }
        setup_shm(pm, ep_count);
        // dial every lower rank that is not reached through shared memory, once per endpoint
        for (int e = 0; e < ep_count; e++) {
            for (int p = 0; p < rank_; p++) {
                if (eps_[e].peers[p].tx)
                    continue;
                int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
                sockaddr_in d{};
                d.sin_family = AF_INET;
                d.sin_port = htons((uint16_t)table[p].port);
                const char* dip = same_host_[p] ? "127.0.0.1" : table[p].ip;
                inet_pton(AF_INET, dip, &d.sin_addr);
                int tries = 0;
                while (::connect(fd, (sockaddr*)&d, sizeof(d)) != 0) {
                    CCL_THROW_IF_NOT(++tries < 2000, "can not connect to rank ", p, " at ", dip, ":", table[p].port,
                                     ": ", std::strerror(errno));
                    usleep(5000);
                }
                int hello[2] = { rank_, e };
                CCL_THROW_IF_NOT(write_blocking(fd, hello, sizeof(hello)), "hello failed");
                eps_[e].peers[p].fd = fd;
            }
        }
        // accept every higher rank
        int expect = 0;
        for (int p = rank_ + 1; p < size_; p++)
            if (!eps_[0].peers[p].tx)
                expect += ep_count;
        for (int i = 0; i < expect; i++) {
            int fd = ::accept4(lfd, nullptr, nullptr, SOCK_CLOEXEC);
            CCL_THROW_IF_NOT(fd >= 0, "accept failed: ", std::strerror(errno));
            int hello[2];
            CCL_THROW_IF_NOT(read_blocking(fd, hello, sizeof(hello)), "hello read failed");
            CCL_THROW_IF_NOT(hello[0] > rank_ && hello[0] < size_ && hello[1] >= 0 && hello[1] < ep_count,
                             "unexpected hello");
            eps_[hello[1]].peers[hello[0]].fd = fd;
        }
        ::close(lfd);
        for (auto& ep : eps_) {
            for (int p = 0; p < size_; p++) {
                if (p == rank_ || ep.peers[p].tx)
                    continue;
                set_nonblock(ep.peers[p].fd);
                epoll_event ev{};
                ev.events = EPOLLIN;
                ev.data.u32 = (uint32_t)p;
                epoll_ctl(ep.epfd, EPOLL_CTL_ADD, ep.peers[p].fd, &ev);
            }
        }
        pm.barrier();
        LOG_DEBUG("mesh transport up: rank ", rank_, "/", size_, ", endpoints ", ep_count, ", shared-memory peers ",
                  eps_[0].shm_peers.size());
    }

    ~tcp_transport() override {
        for (auto& ep : eps_) {
            for (auto& p : ep.peers)
                if (p.fd >= 0)
                    ::close(p.fd);
            if (ep.epfd >= 0)
                ::close(ep.epfd);
        }
        for (auto& m : maps_)
            ::munmap(m.first, m.second);
    }

    int world_rank() const override { return rank_; }
    int world_size() const override { return size_; }
    int ep_count() const override { return (int)eps_.size(); }
    bool same_host(int peer) const override { return same_host_[peer]; }
    const char* name() const override { return eps_[0].shm_peers.empty() ? "tcp" : "shm+tcp"; }

    void send(int e, const void* buf, size_t len, int dst, uint64_t tag, atl_req* req, bool one_way) override {
        endpoint& ep = eps_[e];
        std::lock_guard<std::mutex> lk(ep.mu);
        req->reset();
        msgs_sent++;
        bytes_sent += len;
        peer_state& ps = ep.peers[dst];
        if (dst == rank_) {
            deliver_local(ps, (const char*)buf, len, tag);
            req->done.store(1, std::memory_order_release);
            return;
        }
        if (ps.dead) {
            fail(req);
            return;
        }
        // one-way streams catch up with the rings only above the ring capacity
        if (rndv_min_ && len >= rndv_min_ && same_host_[dst] && (!one_way || len >= ring_cap_)) {
            rndv_sends++;
            ps.awaiting_ack.push_back(req);
            ps.outq.emplace_back();
            out_msg& m = ps.outq.back();
            rndv_desc d{};
            d.addr = (uint64_t)(uintptr_t)buf;
            d.cookie = (uint64_t)(uintptr_t)req;
            d.pid = (int32_t)getpid();
            m.owned.assign((const char*)&d, (const char*)&d + sizeof(d));
            m.hdr.tag = tag;
            m.hdr.len = RNDV_FLAG | (uint64_t)len;
            m.payload = m.owned.data();
            m.payload_len = sizeof(d);
            m.req = nullptr; // the acknowledgement completes the request, not the departure of the descriptor
            flush(ps);
            return;
        }
        out_msg m;
        m.hdr.tag = tag;
        m.hdr.len = len;
        m.payload = (const char*)buf;
        m.payload_len = len;
        m.req = req;
        ps.outq.push_back(m);
        flush(ps);
    }

    void recv(int e, void* buf, size_t len, int src, uint64_t tag, atl_req* req) override {
        endpoint& ep = eps_[e];
        std::lock_guard<std::mutex> lk(ep.mu);
        req->reset();
        peer_state& ps = ep.peers[src];
        for (auto it = ps.unexp.begin(); it != ps.unexp.end(); ++it) {
            if (it->tag != tag)
                continue;
            if (!it->complete) {
                // still arriving: redirect the rest into the user buffer
                CCL_THROW_IF_NOT(it->data.size() <= len, "receive buffer too small: ", len, " < ", it->data.size());
                std::memcpy(buf, it->data.data(), ps.in_got);
                ps.in_dst = (char*)buf;
                ps.in_req = req;
                ps.in_unexp = nullptr;
                req->bytes = it->data.size();
                ps.unexp.erase(it);
                return;
            }
            CCL_THROW_IF_NOT(it->size() <= len, "receive buffer too small: ", len, " < ", it->size());
            if (it->rndv) {
                const rndv_desc d = it->desc;
                const size_t n = it->size();
                ps.unexp.erase(it);
                pull_rendezvous(ps, d, n, (char*)buf, req);
                return;
            }
            std::memcpy(buf, it->data.data(), it->data.size());
            req->bytes = it->data.size();
            bytes_received += it->data.size();
            ps.unexp.erase(it);
            req->done.store(1, std::memory_order_release);
            return;
        }
        if (ps.dead) {
            fail(req);
            return;
        }
        ps.posted.push_back(posted_recv{ tag, (char*)buf, len, req });
    }

    atl_mr mr_reg(void* buf, size_t len) override {
        std::lock_guard<std::mutex> lk(mr_mu_);
        regions_.emplace_back((char*)buf, len);
        atl_mr mr;
        mr.addr = (uint64_t)(uintptr_t)buf;
        mr.len = len;
        mr.pid = (int32_t)getpid();
        mr.owner = rank_;
        return mr;
    }

    void mr_dereg(const atl_mr& mr) override {
        std::lock_guard<std::mutex> lk(mr_mu_);
        for (auto it = regions_.begin(); it != regions_.end(); ++it)
            if ((uint64_t)(uintptr_t)it->first == mr.addr && it->second == mr.len) {
                regions_.erase(it);
                return;
            }
    }

    void rma_write(int e, const void* buf, size_t len, const atl_mr& mr, uint64_t offset, atl_req* req) override {
        CCL_THROW_IF_NOT(mr.owner >= 0 && mr.owner < size_, "one-sided write to an unknown region");
        CCL_THROW_IF_NOT(offset + len <= mr.len, "one-sided write of ", len, " bytes at offset ", offset,
                         " leaves the region of ", mr.len, " bytes");
        req->reset();
        if (mr.owner == rank_) {
            std::memcpy((char*)(uintptr_t)mr.addr + offset, buf, len);
            req->done.store(1, std::memory_order_release);
            return;
        }
        if (same_host_[mr.owner] && env_data::get().atl_cma && cma_ok_.load(std::memory_order_relaxed)) {
            // cross-memory copy into the owner's address space: complete when the call returns
            size_t done = 0;
            bool failed = false;
            while (done < len) {
                iovec l{ (char*)buf + done, len - done };
                iovec r{ (char*)(uintptr_t)mr.addr + offset + done, len - done };
                const ssize_t n = process_vm_writev(mr.pid, &l, 1, &r, 1, 0);
                if (n <= 0) {
                    failed = true;
                    break;
                }
                done += (size_t)n;
            }
            if (!failed) {
                rma_direct_writes++;
                req->done.store(1, std::memory_order_release);
                return;
            }
            CCL_THROW_IF_NOT(done == 0, "cross-memory write stopped after ", done, " of ", len, " bytes: ",
                             std::strerror(errno));
            // not permitted here (ptrace policy, container): every later write goes as a message
            LOG_INFO("process_vm_writev: ", std::strerror(errno), "; one-sided writes travel as messages");
            cma_ok_.store(false, std::memory_order_relaxed);
        }
        endpoint& ep = eps_[e];
        std::lock_guard<std::mutex> lk(ep.mu);
        peer_state& ps = ep.peers[mr.owner];
        rma_message_writes++;
        ps.outq.emplace_back();
        out_msg& m = ps.outq.back();
        m.owned.resize(sizeof(uint64_t) + len);
        const uint64_t target = mr.addr + offset;
        std::memcpy(m.owned.data(), &target, sizeof(target));
        std::memcpy(m.owned.data() + sizeof(target), buf, len);
        m.hdr.tag = RMA_WRITE_TAG;
        m.hdr.len = m.owned.size();
        m.payload = m.owned.data();
        m.payload_len = m.owned.size();
        m.req = req;
        flush(ps);
    }

    bool probe(int e, int src, uint64_t tag, size_t* len) override {
        endpoint& ep = eps_[e];
        std::lock_guard<std::mutex> lk(ep.mu);
        progress(ep);
        for (auto& u : ep.peers[src].unexp)
            if (u.tag == tag && u.complete) {
                if (len)
                    *len = u.size();
                return true;
            }
        return false;
    }

    void poll(int e) override {
        endpoint& ep = eps_[e];
        std::lock_guard<std::mutex> lk(ep.mu);
        progress(ep);
    }

private:
    static size_t ring_stride(size_t cap) { return (shm_ring::footprint(cap) + 4095) & ~(size_t)4095; }
    shm_ring* ring_at(void* seg, int e, int sender) const {
        return (shm_ring*)((char*)seg + ((size_t)e * size_ + sender) * ring_stride(ring_cap_));
    }

    // Shared-memory links to the ranks of this host.  Every rank creates its own segment (the rings
    // it reads from), all ranks agree that creation worked everywhere, then map one another's.
    void setup_shm(pmi& pm, int ep_count) {
        const env_data& env = env_data::get();
        int local_peers = 0;
        for (int r = 0; r < size_; r++)
            local_peers += (r != rank_ && same_host_[r]) ? 1 : 0;
        const bool want = (env.atl_shm || env.atl_transport == atl_transport_t::shm) && size_ > 1;
        ring_cap_ = 64 * 1024;
        while (ring_cap_ * 2 <= env.atl_shm_ring_bytes)
            ring_cap_ *= 2;
        const size_t seg_bytes = (size_t)ep_count * size_ * ring_stride(ring_cap_);
        struct info {
            int ok;
            char name[60];
        } mine{}, zero{};
        void* my_seg = nullptr;
        if (want && local_peers > 0) {
            std::snprintf(mine.name, sizeof(mine.name), "/cclx-%d-%d-%llx", (int)getpid(), rank_,
                          (unsigned long long)std::hash<std::string>()(pm.ns()) & 0xffffffffull);
            int fd = ::shm_open(mine.name, O_CREAT | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
            if (fd >= 0) {
                if (::ftruncate(fd, (off_t)seg_bytes) == 0) {
                    // populated up front: a ring whose pages are touched for the first time costs a page fault per
                    // 4 KiB on both sides, which made 16 KiB messages take 22 us instead of 14 until the whole ring
                    // had been walked once (hundreds of operations)
                    my_seg = ::mmap(nullptr, seg_bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, 0);
                    if (my_seg == MAP_FAILED)
                        my_seg = nullptr;
                }
                ::close(fd);
                if (!my_seg)
                    ::shm_unlink(mine.name);
            }
            mine.ok = my_seg ? 1 : 0;
            if (!my_seg)
                LOG_WARN("shared-memory segment could not be created (", std::strerror(errno), "): sockets only");
        }
        else
            mine.ok = want ? 1 : 0; // nothing to create, nothing against it
        std::vector<info> all(size_, zero);
        pm.allgather(&mine, all.data(), sizeof(info));
        bool everyone = want;
        for (auto& i : all)
            everyone = everyone && i.ok;
        if (my_seg)
            maps_.push_back({ my_seg, seg_bytes });
        if (everyone && my_seg) {
            for (int p = 0; p < size_; p++) {
                if (p == rank_ || !same_host_[p])
                    continue;
                int fd = ::shm_open(all[p].name, O_RDWR | O_CLOEXEC, 0600);
                CCL_THROW_IF_NOT(fd >= 0, "can not open the shared-memory segment of rank ", p, ": ",
                                 std::strerror(errno));
                void* seg = ::mmap(nullptr, seg_bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, 0);
                ::close(fd);
                CCL_THROW_IF_NOT(seg != MAP_FAILED, "can not map the shared-memory segment of rank ", p);
                maps_.push_back({ seg, seg_bytes });
                for (int e = 0; e < ep_count; e++) {
                    eps_[e].peers[p].tx = ring_at(seg, e, rank_);
                    eps_[e].peers[p].rx = ring_at(my_seg, e, p);
                    eps_[e].shm_peers.push_back(p);
                }
            }
        }
        pm.barrier(); // every mapping exists: the names can go, the memory stays until the last unmap
        if (my_seg)
            ::shm_unlink(mine.name);
    }

    // bytes moved (0 = would block); throws on a broken socket
    size_t link_write(peer_state& ps, const void* a, size_t na, const void* b, size_t nb) {
        if (ps.tx) {
            size_t w = ps.tx->write(a, na, ring_cap_);
            if (w == na && nb)
                w += ps.tx->write(b, nb, ring_cap_);
            return w;
        }
        for (;;) {
            iovec iov[2];
            iov[0].iov_base = const_cast<void*>(a);
            iov[0].iov_len = na;
            iov[1].iov_base = const_cast<void*>(b);
            iov[1].iov_len = nb;
            msghdr mh{};
            mh.msg_iov = iov;
            mh.msg_iovlen = nb ? 2 : 1;
            ssize_t r = ::sendmsg(ps.fd, &mh, MSG_NOSIGNAL);
            if (r >= 0)
                return (size_t)r;
            if (errno == EAGAIN || errno == EWOULDBLOCK)
                return 0;
            if (errno == EINTR)
                continue;
            if (errno == EPIPE || errno == ECONNRESET) {
                ps.closed = true;
                return 0;
            }
            CCL_THROW("tcp transport: send failed: ", std::strerror(errno));
        }
    }
    size_t link_read(peer_state& ps, void* dst, size_t n) {
        if (ps.rx)
            return ps.rx->read(dst, n, ring_cap_);
        for (;;) {
            ssize_t r = ::recv(ps.fd, dst, n, 0);
            if (r > 0)
                return (size_t)r;
            if (r == 0) {
                ps.closed = true; // end of stream: the peer exited or closed its transport
                return 0;
            }
            if (errno == EAGAIN || errno == EWOULDBLOCK)
                return 0;
            if (errno == EINTR)
                continue;
            if (errno == ECONNRESET) {
                ps.closed = true;
                return 0;
            }
            CCL_THROW("tcp transport: recv failed: ", std::strerror(errno));
        }
    }

    void deliver_local(peer_state& ps, const char* buf, size_t len, uint64_t tag) {
        for (auto it = ps.posted.begin(); it != ps.posted.end(); ++it) {
            if (it->tag == tag) {
                CCL_THROW_IF_NOT(len <= it->cap, "receive buffer too small");
                std::memcpy(it->buf, buf, len);
                it->req->bytes = len;
                it->req->done.store(1, std::memory_order_release);
                ps.posted.erase(it);
                return;
            }
        }
        ps.unexp.emplace_back();
        unexpected_msg& u = ps.unexp.back();
        u.tag = tag;
        u.data.assign(buf, buf + len);
        u.complete = true;
        unexpected_msgs++;
    }

    void flush(peer_state& ps) {
        while (!ps.outq.empty()) {
            out_msg& m = ps.outq.front();
            const size_t total = sizeof(wire_header) + m.payload_len;
            while (m.sent < total) {
                size_t w;
                if (m.sent < sizeof(wire_header))
                    w = link_write(ps, (char*)&m.hdr + m.sent, sizeof(wire_header) - m.sent, m.payload, m.payload_len);
                else {
                    const size_t off = m.sent - sizeof(wire_header);
                    w = link_write(ps, m.payload + off, m.payload_len - off, nullptr, 0);
                }
                if (w == 0)
                    return;
                m.sent += w;
            }
            if (m.req)
                m.req->done.store(1, std::memory_order_release);
            ps.outq.pop_front();
        }
    }

    // copies a rendezvous message out of the sender's memory and acknowledges it
    void pull_rendezvous(peer_state& ps, const rndv_desc& d, size_t len, char* dst, atl_req* req) {
        size_t done = 0;
        while (done < len) {
            iovec l{ dst + done, len - done };
            iovec r{ (char*)(uintptr_t)d.addr + done, len - done };
            const ssize_t n = process_vm_readv(d.pid, &l, 1, &r, 1, 0);
            if (n <= 0 && errno == ESRCH) { // the sender died after its descriptor left
                fail(req);
                return;
            }
            CCL_THROW_IF_NOT(n > 0, "cross-memory read of ", len, " bytes from process ", d.pid, " failed: ",
                             std::strerror(errno), " (CCL_ATL_CMA=0 sends long messages through the rings)");
            done += (size_t)n;
        }
        bytes_received += len;
        req->bytes = len;
        req->done.store(1, std::memory_order_release);
        ps.outq.emplace_back();
        out_msg& m = ps.outq.back();
        m.owned.assign((const char*)&d.cookie, (const char*)&d.cookie + sizeof(d.cookie));
        m.hdr.tag = RNDV_ACK_TAG;
        m.hdr.len = sizeof(d.cookie);
        m.payload = m.owned.data();
        m.payload_len = sizeof(d.cookie);
        m.req = nullptr;
        flush(ps);
    }

    // a descriptor or an acknowledgement has arrived in ps.ctrl
    void finish_control(peer_state& ps) {
        if (ps.in_hdr.tag == RNDV_ACK_TAG && !(ps.in_hdr.len & RNDV_FLAG)) {
            uint64_t cookie;
            std::memcpy(&cookie, ps.ctrl, sizeof(cookie));
            atl_req* req = (atl_req*)(uintptr_t)cookie;
            auto it = std::find(ps.awaiting_ack.begin(), ps.awaiting_ack.end(), req);
            if (it != ps.awaiting_ack.end()) { // a request that was failed meanwhile is no longer listed
                ps.awaiting_ack.erase(it);
                req->done.store(1, std::memory_order_release);
            }
            return;
        }
        rndv_desc d;
        std::memcpy(&d, ps.ctrl, sizeof(d));
        const size_t len = (size_t)(ps.in_hdr.len & ~RNDV_FLAG);
        for (auto it = ps.posted.begin(); it != ps.posted.end(); ++it) {
            if (it->tag != ps.in_hdr.tag)
                continue;
            CCL_THROW_IF_NOT(len <= it->cap, "receive buffer too small: ", it->cap, " < ", len);
            char* dst = it->buf;
            atl_req* req = it->req;
            ps.posted.erase(it);
            pull_rendezvous(ps, d, len, dst, req);
            return;
        }
        ps.unexp.emplace_back();
        unexpected_msg& u = ps.unexp.back();
        u.tag = ps.in_hdr.tag;
        u.rndv = true;
        u.rndv_len = len;
        u.desc = d;
        u.complete = true;
        unexpected_msgs++;
    }

    void finish_incoming(peer_state& ps) {
        if (ps.in_ctrl) {
            ps.in_ctrl = false;
            ps.in_dst = nullptr;
            ps.in_body = false;
            ps.hdr_got = 0;
            ps.in_got = 0;
            finish_control(ps);
            return;
        }
        bytes_received += ps.in_hdr.len;
        if (ps.in_req) {
            ps.in_req->done.store(1, std::memory_order_release);
            ps.in_req = nullptr;
        }
        else if (ps.in_unexp && ps.in_unexp->tag == RMA_WRITE_TAG) {
            apply_remote_write(ps.in_unexp->data);
            ps.unexp.pop_back(); // the message under construction is always the last one
        }
        else if (ps.in_unexp)
            ps.in_unexp->complete = true;
        ps.in_unexp = nullptr;
        ps.in_dst = nullptr;
        ps.in_body = false;
        ps.hdr_got = 0;
        ps.in_got = 0;
    }

    // a one-sided write that came as a message: only registered memory is ever written
    void apply_remote_write(const std::vector<char>& msg) {
        if (msg.size() < sizeof(uint64_t))
            return;
        uint64_t target;
        std::memcpy(&target, msg.data(), sizeof(target));
        const size_t len = msg.size() - sizeof(target);
        char* dst = (char*)(uintptr_t)target;
        bool inside = false;
        {
            std::lock_guard<std::mutex> lk(mr_mu_);
            for (auto& r : regions_)
                if (dst >= r.first && dst + len <= r.first + r.second)
                    inside = true;
        }
        if (!inside) {
            LOG_ERROR("dropped a one-sided write of ", len, " bytes outside every registered region");
            return;
        }
        std::memcpy(dst, msg.data() + sizeof(target), len);
        std::atomic_thread_fence(std::memory_order_release);
    }

    void drain(peer_state& ps) {
        for (;;) {
            if (!ps.in_body) {
                const size_t r = link_read(ps, (char*)&ps.in_hdr + ps.hdr_got, sizeof(wire_header) - ps.hdr_got);
                if (r == 0)
                    return;
                ps.hdr_got += r;
                if (ps.hdr_got < sizeof(wire_header))
                    continue;
                // header complete: find where the body goes
                ps.in_body = true;
                ps.in_got = 0;
                ps.in_req = nullptr;
                ps.in_unexp = nullptr;
                const bool rndv = (ps.in_hdr.len & RNDV_FLAG) != 0;
                if (rndv || ps.in_hdr.tag == RNDV_ACK_TAG) {
                    ps.in_ctrl = true;
                    ps.body_len = rndv ? sizeof(rndv_desc) : sizeof(uint64_t);
                    ps.in_dst = ps.ctrl;
                    continue;
                }
                ps.body_len = (size_t)ps.in_hdr.len;
                bool matched = false;
                for (auto it = ps.posted.begin(); it != ps.posted.end(); ++it) {
                    if (it->tag == ps.in_hdr.tag) {
                        CCL_THROW_IF_NOT(ps.in_hdr.len <= it->cap, "receive buffer too small: ", it->cap, " < ",
                                         ps.in_hdr.len);
                        ps.in_dst = it->buf;
                        ps.in_req = it->req;
                        it->req->bytes = ps.in_hdr.len;
                        ps.posted.erase(it);
                        matched = true;
                        break;
                    }
                }
                if (!matched) {
                    ps.unexp.emplace_back();
                    unexpected_msg& u = ps.unexp.back();
                    u.tag = ps.in_hdr.tag;
                    u.data.resize(ps.in_hdr.len);
                    ps.in_dst = u.data.data();
                    ps.in_unexp = &u;
                    unexpected_msgs++;
                }
                if (ps.in_hdr.len == 0) {
                    finish_incoming(ps);
                    continue;
                }
            }
            const size_t r = link_read(ps, ps.in_dst + ps.in_got, ps.body_len - ps.in_got);
            if (r == 0)
                return;
            ps.in_got += r;
            if (ps.in_got == ps.body_len)
                finish_incoming(ps);
        }
    }

    static void fail(atl_req* req) {
        req->error = 1;
        req->done.store(1, std::memory_order_release);
    }

    // Nothing more will come from this peer and nothing can reach it: every operation that waits on it
    // ends with an error, which the schedule turns into an exception on the caller's side.
    void fail_peer(peer_state& ps, int p, const char* why) {
        if (ps.dead)
            return;
        ps.dead = true;
        peers_lost++;
        const size_t pending = ps.posted.size() + ps.outq.size() + ps.awaiting_ack.size();
        if (pending)
            LOG_WARN("rank ", p, " is gone (", why, "): failing ", pending, " pending operation(s)");
        else
            LOG_DEBUG("rank ", p, " is gone (", why, ")");
        for (auto& r : ps.posted)
            fail(r.req);
        ps.posted.clear();
        for (auto& m : ps.outq)
            if (m.req)
                fail(m.req);
        ps.outq.clear();
        for (atl_req* r : ps.awaiting_ack)
            fail(r);
        ps.awaiting_ack.clear();
    }

    static bool process_gone(int pid) {
        if (::kill(pid, 0) != 0)
            return errno == ESRCH;
        // a process that exited but was not reaped yet still has a pid: look at its state
        char path[64], buf[256];
        std::snprintf(path, sizeof(path), "/proc/%d/stat", pid);
        int fd = ::open(path, O_RDONLY | O_CLOEXEC);
        if (fd < 0)
            return false;
        const ssize_t n = ::read(fd, buf, sizeof(buf) - 1);
        ::close(fd);
        if (n <= 0)
            return false;
        buf[n] = 0;
        const char* paren = std::strrchr(buf, ')');
        return paren && (paren[2] == 'Z' || paren[2] == 'X');
    }

    void progress(endpoint& ep) {
        for (auto& ps : ep.peers)
            if (!ps.outq.empty())
                flush(ps);
        for (int p : ep.shm_peers)
            if (ep.peers[p].rx->readable())
                drain(ep.peers[p]);
        // Liveness of the peers behind shared-memory rings (a ring never reports that its other end died):
        // every 100 ms, and only for peers this endpoint is waiting on.  What the peer wrote before it died
        // is still in the ring and is delivered first.
        if (!ep.shm_peers.empty() && (++ep.liveness_tick & 1023) == 0) {
            timespec ts;
            clock_gettime(CLOCK_MONOTONIC, &ts);
            const uint64_t now = (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
            if (now - ep.last_liveness_ns > 100000000ull) {
                ep.last_liveness_ns = now;
                for (int p : ep.shm_peers) {
                    peer_state& ps = ep.peers[p];
                    if (ps.dead || pids_[p] == 0 || (ps.posted.empty() && ps.outq.empty() && ps.awaiting_ack.empty()))
                        continue;
                    if (process_gone(pids_[p])) {
                        drain(ps);
                        fail_peer(ps, p, "its process has exited");
                    }
                }
            }
        }
        if (ep.shm_peers.size() + 1 == ep.peers.size())
            return; // no socket on this endpoint
        epoll_event evs[64];
        int n = epoll_wait(ep.epfd, evs, 64, 0);
        for (int i = 0; i < n; i++) {
            peer_state& ps = ep.peers[evs[i].data.u32];
            drain(ps);
            if (ps.closed && !ps.dead) {
                epoll_ctl(ep.epfd, EPOLL_CTL_DEL, ps.fd, nullptr);
                fail_peer(ps, (int)evs[i].data.u32, "it closed the connection");
            }
        }
        for (auto& ps : ep.peers) // a reset seen while writing
            if (ps.closed && !ps.dead)
                fail_peer(ps, (int)(&ps - &ep.peers[0]), "the connection was reset");
    }

    int rank_, size_;
    std::vector<endpoint> eps_;
    std::vector<char> same_host_;
    size_t ring_cap_ = 0;
    std::vector<std::pair<void*, size_t>> maps_;
    std::mutex mr_mu_;
    std::vector<std::pair<char*, size_t>> regions_;
    std::atomic<bool> cma_ok_{ true };
    std::vector<int> pids_; // of the ranks on this host whose pid is visible here, else 0
    size_t rndv_min_ = 0; // messages of at least this size between processes of one host go by rendezvous (0: never)
};

} // namespace

std::shared_ptr<atl_transport> create_tcp_transport(pmi& pm, int ep_count) {
    return std::make_shared<tcp_transport>(pm, ep_count);
}

// ---- atl_comm ---------------------------------------------------------------------

static std::atomic<uint64_t> g_next_comm_id{ 1 };

uint64_t atl_comm::next_comm_id() {
    return g_next_comm_id.load();
}
void atl_comm::bump_comm_id(uint64_t at_least) {
    uint64_t cur = g_next_comm_id.load();
    while (cur < at_least && !g_next_comm_id.compare_exchange_weak(cur, at_least)) {
    }
}

atl_comm::atl_comm(std::shared_ptr<atl_transport> tr, std::vector<int> world_ranks, int my_index, uint64_t comm_id)
        : tr_(std::move(tr)), ranks_(std::move(world_ranks)), rank_(my_index), comm_id_(comm_id) {}

void atl_comm::wait(int ep, atl_req* req) {
    while (!req->is_done())
        tr_->poll(ep);
    CCL_THROW_IF_NOT(!req->error, "a peer of this communicator has left the job (process gone or connection closed)");
}

void atl_comm::allgather(const void* send_buf, void* recv_buf, size_t n) {
    const int W = size();
    const uint64_t tag = atl_tag::make(comm_id_, atl_tag::INTERNAL_SCHED, internal_op_++ & atl_tag::MAX_OP);
    std::vector<atl_req> sreq(W), rreq(W);
    std::memcpy((char*)recv_buf + (size_t)rank_ * n, send_buf, n);
    for (int p = 0; p < W; p++) {
        if (p == rank_)
            continue;
        recv(0, (char*)recv_buf + (size_t)p * n, n, p, tag, &rreq[p]);
    }
    for (int p = 0; p < W; p++) {
        if (p == rank_)
            continue;
        send(0, send_buf, n, p, tag, &sreq[p]);
    }
    for (int p = 0; p < W; p++) {
        if (p == rank_)
            continue;
        wait(0, &sreq[p]);
        wait(0, &rreq[p]);
    }
}

void atl_comm::barrier() {
    char mine = 1;
    std::vector<char> all(size());
    allgather(&mine, all.data(), 1);
}

std::shared_ptr<atl_comm> atl_comm::split(int color, int key) {
    struct rec {
        int color, key, world_rank;
        uint64_t next_id;
    } mine{ color, key, ranks_[rank_], next_comm_id() };
    std::vector<rec> all(size());
    allgather(&mine, all.data(), sizeof(rec));
    uint64_t base = 0;
    std::vector<int> colors;
    for (auto& r : all) {
        base = std::max(base, r.next_id);
        if (std::find(colors.begin(), colors.end(), r.color) == colors.end())
            colors.push_back(r.color);
    }
    std::sort(colors.begin(), colors.end());
    bump_comm_id(base + colors.size());
    const uint64_t id = base + (uint64_t)(std::find(colors.begin(), colors.end(), color) - colors.begin());
    // members of my color ordered by (key, parent rank)
    std::vector<std::pair<std::pair<int, int>, int>> members; // ((key, parent rank), world rank)
    for (int r = 0; r < size(); r++)
        if (all[r].color == color)
            members.push_back({ { all[r].key, r }, all[r].world_rank });
    std::sort(members.begin(), members.end());
    std::vector<int> wr;
    int me = -1;
    for (size_t i = 0; i < members.size(); i++) {
        wr.push_back(members[i].second);
        if (members[i].first.second == rank_)
            me = (int)i;
    }
    return std::make_shared<atl_comm>(tr_, wr, me, id);
}

} // namespace cclx
