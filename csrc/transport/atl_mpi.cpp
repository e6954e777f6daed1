// MPI transport: the ATL interface on MPI point-to-point messages.
//
// Counterpart of the reference's atl/mpi (src/atl/mpi/atl_mpi.cpp, atl_mpi_comm.cpp) and of its run-time
// loader (src/common/api_wrapper/mpi_api_wrapper.cpp:25-46, entry-point table in mpi_api_wrapper.hpp:26-103):
// the MPI library is opened with dlopen
// (CCL_MPI_LIBRARY_PATH, else libmpi.so.12 / libmpi.so from the loader's search path) and called through the
// MPICH binary interface declared in mpi_abi.hpp.  The processes must have been started by that MPI's launcher,
// so that MPI_COMM_WORLD spans the job; which MPI rank belongs to which rank of the communicator travels through
// the PMI layer, so the two numberings need not agree.
//
// The ATL matches a message by (source, 64-bit tag); MPI tags are ints with as few as 15 usable bits.  So MPI
// carries two kinds of messages per endpoint, each under one fixed MPI tag: a 16-byte header (ATL tag, length)
// and, when the length is not zero, the payload.  Messages of one sender under one MPI tag do not overtake one
// another, so the k-th payload of a sender belongs to its k-th header.  The receiver probes for headers,
// matches them against its posted receives, and receives the payload straight into the user's buffer when a
// receive is waiting, into an unexpected-message buffer otherwise.  poll() drives all of it.
//
// No one-sided writes (CCL_ATL_RMA needs the socket transport).
#include <dlfcn.h>
#include <unistd.h>

#include <climits>
#include <cstdlib>
#include <cstring>
#include <list>
#include <mutex>

#include "bootstrap/pmi.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "transport/atl.hpp"
#include "transport/mpi_abi.hpp"

namespace cclx {

namespace {

using namespace mpiabi;

#define MPI_CALL(expr) \
    do { \
        const int _rc = (expr); \
        if (_rc != SUCCESS) \
            CCL_THROW("MPI: ", #expr, " failed with code ", _rc); \
    } while (0)

library g_lib;

void finalize_at_exit() {
    int fin = 0;
    if (g_lib.handle && g_lib.we_initialised && g_lib.Finalized && g_lib.Finalized(&fin) == SUCCESS && !fin)
        g_lib.Finalize();
}

bool load_library(library& lib, std::string& why) {
    const env_data& env = env_data::get();
    std::vector<std::string> names;
    if (!env.mpi_lib_path.empty())
        names.push_back(env.mpi_lib_path);
    else {
        names.push_back("libmpi.so.12");
        names.push_back("libmpi.so");
    }
    for (auto& n : names) {
        lib.handle = dlopen(n.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (lib.handle)
            break;
        const char* err = dlerror(); // a second call would return null
        why += std::string(err ? err : "dlopen failed") + "; ";
    }
    if (!lib.handle)
        return false;
    if (dlsym(lib.handle, "ompi_mpi_comm_world")) {
        why += "the library is Open MPI, whose binary interface (handles are pointers) differs from the MPICH one this transport speaks";
        dlclose(lib.handle);
        lib.handle = nullptr;
        return false;
    }
    bool all = true;
#define MPI_SYM(field, name) \
    lib.field = (decltype(lib.field))dlsym(lib.handle, name); \
    all = all && lib.field != nullptr
    MPI_SYM(Init_thread, "MPI_Init_thread");
    MPI_SYM(Initialized, "MPI_Initialized");
    MPI_SYM(Finalized, "MPI_Finalized");
    MPI_SYM(Finalize, "MPI_Finalize");
    MPI_SYM(Query_thread, "MPI_Query_thread");
    MPI_SYM(Comm_rank, "MPI_Comm_rank");
    MPI_SYM(Comm_size, "MPI_Comm_size");
    MPI_SYM(Comm_dup, "MPI_Comm_dup");
    MPI_SYM(Comm_free, "MPI_Comm_free");
    MPI_SYM(Isend, "MPI_Isend");
    MPI_SYM(Irecv, "MPI_Irecv");
    MPI_SYM(Recv, "MPI_Recv");
    MPI_SYM(Test, "MPI_Test");
    MPI_SYM(Iprobe, "MPI_Iprobe");
    MPI_SYM(Get_count, "MPI_Get_count");
#undef MPI_SYM
    lib.Get_library_version = (decltype(lib.Get_library_version))dlsym(lib.handle, "MPI_Get_library_version");
    if (!all) {
        why += "MPI entry points missing";
        dlclose(lib.handle);
        lib.handle = nullptr;
        return false;
    }
    return true;
}

struct wire_header {
    uint64_t tag;
    uint64_t len;
};

class mpi_transport : public atl_transport {
public:
    mpi_transport(pmi& pm, int ep_count, library lib, int thread_level)
            : lib_(lib), rank_(pm.rank()), size_(pm.size()), serial_(thread_level < THREAD_MULTIPLE), eps_(ep_count) {
        MPI_CALL(lib_.Comm_dup(COMM_WORLD, &comm_));
        int mine = -1;
        MPI_CALL(lib_.Comm_rank(comm_, &mine));
        mpi_rank_.assign(size_, -1);
        pm.allgather(&mine, mpi_rank_.data(), sizeof(int));
        of_mpi_rank_.assign(size_, -1);
        for (int r = 0; r < size_; r++) {
            CCL_THROW_IF_NOT(mpi_rank_[r] >= 0 && mpi_rank_[r] < size_ && of_mpi_rank_[mpi_rank_[r]] < 0,
                             "the ranks' MPI ranks are not a permutation of 0 .. ", size_ - 1);
            of_mpi_rank_[mpi_rank_[r]] = r;
        }
        char host[64] = { 0 };
        gethostname(host, sizeof(host) - 1);
        std::vector<char> hosts((size_t)size_ * sizeof(host));
        pm.allgather(host, hosts.data(), sizeof(host));
        same_host_.resize(size_);
        for (int r = 0; r < size_; r++)
            same_host_[r] = std::strncmp(hosts.data() + (size_t)r * sizeof(host), host, sizeof(host)) == 0;
        name_ = "mpi";
        if (lib_.Get_library_version) {
            char v[8192] = { 0 };
            int n = 0;
            if (lib_.Get_library_version(v, &n) == SUCCESS) {
                std::string s(v);
                s = s.substr(0, s.find('\n'));
                LOG_INFO("mpi transport: ", s, ", ", ep_count, " endpoint(s), thread level ", thread_level);
            }
        }
        pm.barrier();
    }

    ~mpi_transport() override {
        int fin = 0;
        if (lib_.Finalized(&fin) == SUCCESS && !fin)
            lib_.Comm_free(&comm_);
    }

    int world_rank() const override { return rank_; }
    int world_size() const override { return size_; }
    int ep_count() const override { return (int)eps_.size(); }
    bool same_host(int peer) const override { return same_host_[peer]; }
    const char* name() const override { return name_.c_str(); }

    void send(int e, const void* buf, size_t len, int dst, uint64_t tag, atl_req* req, bool) override {
        const int ei = e % (int)eps_.size();
        endpoint& ep = eps_[ei];
        req->reset();
        bytes_sent += len;
        msgs_sent++;
        CCL_THROW_IF_NOT(len <= (size_t)INT_MAX, "a message of ", len,
                         " bytes exceeds the count of one MPI message (CCL_ATL_LARGE_MSG_SIZE splits larger operations)");
        std::lock_guard<std::mutex> lk(ep.mu);
        if (dst == rank_) {
            self_send(ep, buf, len, tag, req);
            return;
        }
        out_msg* o = new out_msg();
        o->hdr = wire_header{ tag, (uint64_t)len };
        o->req = req;
        big_lock g(*this);
        MPI_CALL(lib_.Isend(&o->hdr, (int)sizeof(wire_header), BYTE, mpi_rank_[dst], 2 * ei, comm_, &o->mpi[0]));
        o->n = 1;
        if (len) {
            MPI_CALL(lib_.Isend(buf, (int)len, BYTE, mpi_rank_[dst], 2 * ei + 1, comm_, &o->mpi[1]));
            o->n = 2;
        }
        ep.sends.push_back(o);
    }

    void recv(int e, void* buf, size_t len, int src, uint64_t tag, atl_req* req) override {
        endpoint& ep = eps_[e % (int)eps_.size()];
        req->reset();
        std::lock_guard<std::mutex> lk(ep.mu);
        if (src == rank_) {
            self_recv(ep, buf, len, tag, req);
            return;
        }
        for (auto it = ep.unexpected.begin(); it != ep.unexpected.end(); ++it)
            if (it->src == src && it->tag == tag && !it->waiter) {
                if (it->arrived) {
                    deliver(*it, buf, len, req);
                    ep.unexpected.erase(it);
                }
                else { // the payload is still on its way into the buffer: finish when it is there
                    it->waiter = req;
                    it->wbuf = buf;
                    it->wlen = len;
                }
                return;
            }
        ep.posted.push_back(posted_recv{ src, tag, buf, len, req });
    }

    bool probe(int e, int src, uint64_t tag, size_t* len) override {
        const int ei = e % (int)eps_.size();
        endpoint& ep = eps_[ei];
        std::lock_guard<std::mutex> lk(ep.mu);
        if (src == rank_) {
            for (auto& m : ep.self_unexpected)
                if (m.tag == tag) {
                    if (len)
                        *len = m.data.size();
                    return true;
                }
            return false;
        }
        progress(ep, ei);
        for (auto& u : ep.unexpected)
            if (u.src == src && u.tag == tag && !u.waiter) {
                if (len)
                    *len = u.data.size();
                return true;
            }
        return false;
    }

    void poll(int e) override {
        const int ei = e % (int)eps_.size();
        endpoint& ep = eps_[ei];
        std::unique_lock<std::mutex> lk(ep.mu, std::try_to_lock);
        if (!lk.owns_lock())
            return;
        progress(ep, ei);
    }

    bool has_rma() const override { return false; }
    atl_mr mr_reg(void*, size_t) override {
        CCL_THROW("one-sided writes are not offered by the mpi transport (use the socket transport for CCL_ATL_RMA)");
    }
    void mr_dereg(const atl_mr&) override {}
    void rma_write(int, const void*, size_t, const atl_mr&, uint64_t, atl_req*) override {
        CCL_THROW("one-sided writes are not offered by the mpi transport");
    }

private:
    struct out_msg {
        wire_header hdr;
        request_t mpi[2];
        int n = 0;
        atl_req* req = nullptr;
    };
    struct posted_recv {
        int src;
        uint64_t tag;
        void* buf;
        size_t len;
        atl_req* req;
    };
    struct unexpected_msg {
        int src;
        uint64_t tag;
        std::vector<char> data;
        bool arrived = false;
        atl_req* waiter = nullptr; // a receive that was posted while the payload was arriving
        void* wbuf = nullptr;
        size_t wlen = 0;
    };
    struct incoming {
        request_t mpi;
        atl_req* req; // direct delivery into a posted buffer, else null
        size_t len;
        unexpected_msg* unexp; // delivery into an unexpected-message buffer, else null
    };
    struct self_msg {
        uint64_t tag;
        std::vector<char> data;
    };
    struct endpoint {
        std::mutex mu;
        std::list<out_msg*> sends;
        std::list<posted_recv> posted;
        std::list<unexpected_msg> unexpected; // std::list: `incoming` keeps pointers to its elements
        std::list<incoming> arriving;
        std::list<self_msg> self_unexpected;
        std::list<posted_recv> self_recvs;
    };
    // below MPI_THREAD_MULTIPLE every MPI call of the process is serialised by one lock
    struct big_lock {
        explicit big_lock(mpi_transport& t) : mu(t.serial_ ? &t.big_ : nullptr) {
            if (mu)
                mu->lock();
        }
        ~big_lock() {
            if (mu)
                mu->unlock();
        }
        std::mutex* mu;
    };

    void deliver(unexpected_msg& u, void* buf, size_t len, atl_req* req) {
        const size_t n = std::min(len, u.data.size());
        if (n)
            std::memcpy(buf, u.data.data(), n);
        req->bytes = n;
        bytes_received += n;
        req->done.store(1, std::memory_order_release);
    }

    void progress(endpoint& ep, int ei) {
        big_lock g(*this);
        // sends: both messages handed over
        for (auto it = ep.sends.begin(); it != ep.sends.end();) {
            out_msg* o = *it;
            bool all = true;
            for (int k = 0; k < o->n; k++) {
                if (o->mpi[k] == REQUEST_NULL)
                    continue;
                int flag = 0;
                MPI_CALL(lib_.Test(&o->mpi[k], &flag, (status_t*)1 /* MPI_STATUS_IGNORE */));
                if (flag)
                    o->mpi[k] = REQUEST_NULL;
                else
                    all = false;
            }
            if (all) {
                o->req->done.store(1, std::memory_order_release);
                delete o;
                it = ep.sends.erase(it);
            }
            else
                ++it;
        }
        // new headers
        for (int budget = 0; budget < 64; budget++) {
            int flag = 0;
            status_t st{};
            MPI_CALL(lib_.Iprobe(ANY_SOURCE, 2 * ei, comm_, &flag, &st));
            if (!flag)
                break;
            wire_header h{};
            MPI_CALL(lib_.Recv(&h, (int)sizeof(h), BYTE, st.source, 2 * ei, comm_, (status_t*)1));
            const int src = of_mpi_rank_[st.source];
            auto p = ep.posted.begin();
            for (; p != ep.posted.end(); ++p)
                if (p->src == src && p->tag == h.tag)
                    break;
            if (p != ep.posted.end() && p->len >= h.len) {
                if (h.len == 0) {
                    p->req->bytes = 0;
                    p->req->done.store(1, std::memory_order_release);
                }
                else {
                    incoming in{ REQUEST_NULL, p->req, (size_t)h.len, nullptr };
                    MPI_CALL(lib_.Irecv(p->buf, (int)h.len, BYTE, st.source, 2 * ei + 1, comm_, &in.mpi));
                    ep.arriving.push_back(in);
                }
                ep.posted.erase(p);
                continue;
            }
            // nobody waits for it (or waits with a shorter buffer): into a buffer of its own
            ep.unexpected.emplace_back();
            unexpected_msg& u = ep.unexpected.back();
            u.src = src;
            u.tag = h.tag;
            u.data.resize(h.len);
            unexpected_msgs++;
            if (p != ep.posted.end()) { // the shorter receive takes what fits once the payload is there
                u.waiter = p->req;
                u.wbuf = p->buf;
                u.wlen = p->len;
                ep.posted.erase(p);
            }
            if (h.len == 0)
                u.arrived = true;
            else {
                incoming in{ REQUEST_NULL, nullptr, (size_t)h.len, &u };
                MPI_CALL(lib_.Irecv(u.data.data(), (int)h.len, BYTE, st.source, 2 * ei + 1, comm_, &in.mpi));
                ep.arriving.push_back(in);
            }
            if (u.arrived && u.waiter)
                finish_unexpected(ep, u);
        }
        // payloads
        for (auto it = ep.arriving.begin(); it != ep.arriving.end();) {
            int flag = 0;
            MPI_CALL(lib_.Test(&it->mpi, &flag, (status_t*)1));
            if (!flag) {
                ++it;
                continue;
            }
            if (it->req) {
                it->req->bytes = it->len;
                bytes_received += it->len;
                it->req->done.store(1, std::memory_order_release);
            }
            else {
                it->unexp->arrived = true;
                if (it->unexp->waiter)
                    finish_unexpected(ep, *it->unexp);
            }
            it = ep.arriving.erase(it);
        }
    }

    void finish_unexpected(endpoint& ep, unexpected_msg& u) {
        deliver(u, u.wbuf, u.wlen, u.waiter);
        for (auto it = ep.unexpected.begin(); it != ep.unexpected.end(); ++it)
            if (&*it == &u) {
                ep.unexpected.erase(it);
                return;
            }
    }

    void self_send(endpoint& ep, const void* buf, size_t len, uint64_t tag, atl_req* req) {
        for (auto it = ep.self_recvs.begin(); it != ep.self_recvs.end(); ++it)
            if (it->tag == tag) {
                const size_t n = std::min(len, it->len);
                if (n)
                    std::memcpy(it->buf, buf, n);
                it->req->bytes = n;
                it->req->done.store(1, std::memory_order_release);
                ep.self_recvs.erase(it);
                req->done.store(1, std::memory_order_release);
                return;
            }
        ep.self_unexpected.push_back(self_msg{ tag, std::vector<char>((const char*)buf, (const char*)buf + len) });
        unexpected_msgs++;
        req->done.store(1, std::memory_order_release);
    }

    void self_recv(endpoint& ep, void* buf, size_t len, uint64_t tag, atl_req* req) {
        for (auto it = ep.self_unexpected.begin(); it != ep.self_unexpected.end(); ++it)
            if (it->tag == tag) {
                const size_t n = std::min(len, it->data.size());
                if (n)
                    std::memcpy(buf, it->data.data(), n);
                req->bytes = n;
                ep.self_unexpected.erase(it);
                req->done.store(1, std::memory_order_release);
                return;
            }
        ep.self_recvs.push_back(posted_recv{ rank_, tag, buf, len, req });
    }

    library lib_;
    int rank_, size_;
    bool serial_;
    std::mutex big_;
    comm_t comm_ = 0;
    std::vector<int> mpi_rank_, of_mpi_rank_;
    std::vector<endpoint> eps_;
    std::vector<char> same_host_;
    std::string name_;
};

} // namespace

// Null, with the reason in `why`, unless EVERY rank can load an MPI library of the MPICH binary interface whose
// MPI_COMM_WORLD has as many ranks as the communicator (the ranks agree through the PMI layer, so that either all
// of them use it or none does).
std::shared_ptr<atl_transport> create_mpi_transport(pmi& pm, int ep_count, std::string& why) {
    static std::mutex mu;
    static int thread_level = THREAD_SINGLE;
    int ok = 1;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!g_lib.handle) {
            if (!load_library(g_lib, why))
                ok = 0;
            else {
                int init = 0;
                if (g_lib.Initialized(&init) != SUCCESS)
                    ok = 0;
                else if (!init) {
                    if (g_lib.Init_thread(nullptr, nullptr, THREAD_MULTIPLE, &thread_level) != SUCCESS) {
                        why += "MPI_Init_thread failed";
                        ok = 0;
                    }
                    else {
                        g_lib.we_initialised = true;
                        std::atexit(finalize_at_exit);
                    }
                }
                else
                    g_lib.Query_thread(&thread_level);
            }
        }
        if (ok) {
            int n = 0;
            if (g_lib.Comm_size(COMM_WORLD, &n) != SUCCESS || n != pm.size()) {
                why += "MPI_COMM_WORLD has " + std::to_string(n) + " rank(s), the communicator " + std::to_string(pm.size()) +
                       " (the processes must be started by the MPI launcher)";
                ok = 0;
            }
            else if (thread_level < THREAD_SERIALIZED) {
                why += "the MPI library offers thread level " + std::to_string(thread_level) +
                       ", the worker threads need MPI_THREAD_SERIALIZED at least";
                ok = 0;
            }
        }
    }
    std::vector<int> all(pm.size(), 0);
    pm.allgather(&ok, all.data(), sizeof(int));
    for (int r = 0; r < pm.size(); r++)
        if (!all[r]) {
            if (ok)
                why = "rank " + std::to_string(r) + " could not use MPI";
            return nullptr;
        }
    return std::make_shared<mpi_transport>(pm, ep_count, g_lib, thread_level);
}

} // namespace cclx
