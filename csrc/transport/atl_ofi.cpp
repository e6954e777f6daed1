// OFI transport: the ATL interface on libfabric's tagged messages.
//
// Counterpart of the reference's atl/ofi (src/atl/ofi/atl_ofi.cpp:30-1196, atl_ofi_helper.cpp:78-1393) and of
// its run-time loader (src/common/api_wrapper/ofi_api_wrapper.cpp:26-84): libfabric is opened with dlopen
// (CCL_OFI_LIBRARY_PATH, else the loader's search path), a reliable-datagram provider is asked for with
// tagged messages and directed receives, one endpoint with its own completion queue serves every worker,
// the endpoints' names travel through the PMI layer into one address table, and send / recv / probe map to
// fi_tsend / fi_trecv / a peeking fi_trecvmsg.  Completions are reaped by poll(), which is what the workers
// call in their progress loop.  Messages of a rank to itself never reach the provider.
//
// Differences from the socket transport of this library: no shared-memory rings or cross-memory rendezvous
// of its own (the provider decides how bytes move) and no one-sided writes (CCL_ATL_RMA needs the socket
// transport).
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <deque>
#include <list>
#include <map>
#include <mutex>

#include "bootstrap/pmi.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "transport/atl.hpp"
#include "transport/ofi_abi.hpp"

namespace cclx {

namespace {

using namespace ofi;

#define OFI_CALL(expr) \
    do { \
        const long _rc = (long)(expr); \
        if (_rc < 0) \
            CCL_THROW("libfabric: ", #expr, " failed: ", lib_.strerror ? lib_.strerror((int)-_rc) : "?", " (", _rc, ")"); \
    } while (0)

bool load_library(library& lib, std::string& why) {
    const env_data& env = env_data::get();
    std::vector<std::string> names;
    if (!env.ofi_lib_path.empty())
        names.push_back(env.ofi_lib_path);
    else {
        names.push_back("libfabric.so.1");
        names.push_back("libfabric.so");
    }
    for (auto& n : names) {
        // providers that ship as separate objects next to the library (<dir>/prov) are found through
        // FI_PROVIDER_PATH, which the user may have set; point it there otherwise
        if (n.find('/') != std::string::npos && !getenv("FI_PROVIDER_PATH")) {
            const std::string dir = n.substr(0, n.rfind('/')) + "/prov";
            struct stat st;
            if (stat(dir.c_str(), &st) == 0)
                setenv("FI_PROVIDER_PATH", dir.c_str(), 0);
        }
        lib.handle = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (lib.handle)
            break;
        const char* err = dlerror(); // a second call would return null
        why += std::string(err ? err : "dlopen failed") + "; ";
    }
    if (!lib.handle)
        return false;
    lib.getinfo = (decltype(lib.getinfo))dlsym(lib.handle, "fi_getinfo");
    lib.freeinfo = (decltype(lib.freeinfo))dlsym(lib.handle, "fi_freeinfo");
    lib.dupinfo = (decltype(lib.dupinfo))dlsym(lib.handle, "fi_dupinfo");
    lib.fabric = (decltype(lib.fabric))dlsym(lib.handle, "fi_fabric");
    lib.strerror = (decltype(lib.strerror))dlsym(lib.handle, "fi_strerror");
    lib.version = (decltype(lib.version))dlsym(lib.handle, "fi_version");
    if (!lib.getinfo || !lib.freeinfo || !lib.dupinfo || !lib.fabric) {
        why += "libfabric entry points missing";
        dlclose(lib.handle);
        lib.handle = nullptr;
        return false;
    }
    return true;
}

class ofi_transport : public atl_transport {
public:
    ofi_transport(pmi& pm, int ep_count, library lib) : lib_(lib), rank_(pm.rank()), size_(pm.size()), eps_(ep_count) {
        fi_info* hints = lib_.dupinfo(nullptr);
        CCL_THROW_IF_NOT(hints != nullptr, "libfabric: fi_allocinfo failed");
        hints->caps = CAP_TAGGED | CAP_SEND | CAP_RECV | CAP_DIRECTED_RECV;
        hints->mode = MODE_CONTEXT | MODE_CONTEXT2; // every operation carries provider scratch space (op::ctx)
        hints->ep_attr->type = EP_RDM;
        hints->domain_attr->threading = THREAD_SAFE;
        hints->domain_attr->av_type = AV_TABLE;
        hints->domain_attr->resource_mgmt = RM_ENABLED;
        hints->tx_attr->msg_order = ORDER_SAS;
        hints->rx_attr->msg_order = ORDER_SAS;
        // which provider serves the request is libfabric's choice; FI_PROVIDER narrows it as usual
        fi_info* found = nullptr;
        const int rc = lib_.getinfo(make_version(1, 9), nullptr, nullptr, 0, hints, &found);
        lib_.freeinfo(hints);
        if (rc != 0 || !found)
            CCL_THROW("libfabric offers no reliable-datagram provider with tagged messages and directed receives"
                      " (fi_getinfo: ", lib_.strerror ? lib_.strerror(-rc) : "?", ")");
        info_ = found;
        prov_ = info_->fabric_attr && info_->fabric_attr->prov_name ? info_->fabric_attr->prov_name : "?";
        name_ = "ofi:" + prov_;
        OFI_CALL(lib_.fabric(info_->fabric_attr, &fabric_, nullptr));
        OFI_CALL(fabric_->ops->domain(fabric_, info_, &domain_, nullptr));
        fi_av_attr av_attr{};
        av_attr.type = AV_TABLE;
        av_attr.count = (size_t)size_ * ep_count;
        OFI_CALL(domain_->ops->av_open(domain_, &av_attr, &av_, nullptr));

        constexpr size_t NAME_MAX_BYTES = 128;
        std::vector<char> mine((size_t)ep_count * NAME_MAX_BYTES, 0);
        for (int e = 0; e < ep_count; e++) {
            endpoint& ep = eps_[e];
            fi_cq_attr cq_attr{};
            cq_attr.format = CQ_FORMAT_TAGGED;
            cq_attr.wait_obj = WAIT_NONE;
            cq_attr.size = 4096;
            OFI_CALL(domain_->ops->cq_open(domain_, &cq_attr, &ep.cq, nullptr));
            OFI_CALL(domain_->ops->endpoint(domain_, info_, &ep.ep, nullptr));
            OFI_CALL(ep.ep->f.ops->bind(&ep.ep->f, &ep.cq->f, CAP_SEND | CAP_RECV));
            OFI_CALL(ep.ep->f.ops->bind(&ep.ep->f, &av_->f, 0));
            OFI_CALL(ep.ep->f.ops->control(&ep.ep->f, CTRL_ENABLE, nullptr));
            size_t len = NAME_MAX_BYTES;
            OFI_CALL(ep.ep->cm->getname(&ep.ep->f, mine.data() + (size_t)e * NAME_MAX_BYTES, &len));
            CCL_THROW_IF_NOT(len <= NAME_MAX_BYTES, "libfabric endpoint name of ", len, " bytes is longer than expected");
        }
        // address table through the PMI layer: entry (e, r) = endpoint e of rank r
        std::vector<char> all((size_t)size_ * mine.size());
        pm.allgather(mine.data(), all.data(), mine.size());
        for (int e = 0; e < ep_count; e++) {
            eps_[e].peer.assign(size_, ADDR_UNSPEC);
            for (int r = 0; r < size_; r++) {
                fi_addr_t a = ADDR_UNSPEC;
                const int n = av_->ops->insert(av_, all.data() + (size_t)r * mine.size() + (size_t)e * NAME_MAX_BYTES, 1,
                                               &a, 0, nullptr);
                CCL_THROW_IF_NOT(n == 1, "libfabric: fi_av_insert failed for rank ", r);
                eps_[e].peer[r] = a;
            }
        }
        char host[64] = { 0 };
        gethostname(host, sizeof(host) - 1);
        std::vector<char> hosts((size_t)size_ * sizeof(host));
        pm.allgather(host, hosts.data(), sizeof(host));
        same_host_.resize(size_);
        for (int r = 0; r < size_; r++)
            same_host_[r] = std::strncmp(hosts.data() + (size_t)r * sizeof(host), host, sizeof(host)) == 0;
        pm.barrier(); // every endpoint exists before the first message leaves
        LOG_INFO("ofi transport: provider ", prov_, ", ", ep_count, " endpoint(s), libfabric ",
                 lib_.version ? (int)(lib_.version() >> 16) : 0, ".", lib_.version ? (int)(lib_.version() & 0xffff) : 0);
    }

    ~ofi_transport() override {
        for (auto& ep : eps_) {
            if (ep.ep)
                ep.ep->f.ops->close(&ep.ep->f);
            if (ep.cq)
                ep.cq->f.ops->close(&ep.cq->f);
        }
        if (av_)
            av_->f.ops->close(&av_->f);
        if (domain_)
            domain_->f.ops->close(&domain_->f);
        if (fabric_)
            fabric_->f.ops->close(&fabric_->f);
        if (info_)
            lib_.freeinfo(info_);
        // the library stays loaded: providers may have registered exit handlers
    }

    int world_rank() const override { return rank_; }
    int world_size() const override { return size_; }
    int ep_count() const override { return (int)eps_.size(); }
    bool same_host(int peer) const override { return same_host_[peer]; }
    const char* name() const override { return name_.c_str(); }

    void send(int e, const void* buf, size_t len, int dst, uint64_t tag, atl_req* req, bool) override {
        endpoint& ep = eps_[e % eps_.size()];
        req->reset();
        bytes_sent += len;
        msgs_sent++;
        std::lock_guard<std::mutex> lk(ep.mu);
        if (dst == rank_) {
            self_send(ep, buf, len, tag, req);
            return;
        }
        op* o = new op{ {}, req, false, buf, nullptr, len, dst, tag };
        if (!post(ep, o))
            ep.backlog.push_back(o);
    }

    void recv(int e, void* buf, size_t len, int src, uint64_t tag, atl_req* req) override {
        endpoint& ep = eps_[e % eps_.size()];
        req->reset();
        std::lock_guard<std::mutex> lk(ep.mu);
        if (src == rank_) {
            self_recv(ep, buf, len, tag, req);
            return;
        }
        op* o = new op{ {}, req, true, nullptr, buf, len, src, tag };
        if (!post(ep, o))
            ep.backlog.push_back(o);
    }

    // a peeking receive is posted once per (source, tag); its completion says whether the message is there
    bool probe(int e, int src, uint64_t tag, size_t* len) override {
        endpoint& ep = eps_[e % eps_.size()];
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
        const auto key = std::make_pair(src, tag);
        auto it = ep.peeks.find(key);
        if (it == ep.peeks.end()) {
            peek_state* ps = new peek_state();
            ps->o = op{ {}, nullptr, true, nullptr, nullptr, 0, src, tag };
            ps->o.peek = ps;
            fi_msg_tagged m{};
            m.addr = ep.peer[src];
            m.tag = tag;
            m.context = &ps->o.ctx;
            const ssize_t rc = ep.ep->tagged->recvmsg(ep.ep, &m, FLAG_PEEK);
            if (rc == -E_AGAIN) {
                delete ps;
                reap(ep);
                return false;
            }
            OFI_CALL(rc);
            ep.peeks[key] = ps;
            reap(ep);
            it = ep.peeks.find(key);
        }
        else
            reap(ep);
        peek_state* ps = it->second;
        if (ps->state == 0)
            return false;
        const bool found = ps->state == 1;
        if (found && len)
            *len = ps->len;
        delete ps;
        ep.peeks.erase(it);
        return found;
    }

    void poll(int e) override {
        endpoint& ep = eps_[e % eps_.size()];
        std::unique_lock<std::mutex> lk(ep.mu, std::try_to_lock);
        if (!lk.owns_lock())
            return;
        reap(ep);
        while (!ep.backlog.empty()) { // operations the provider had no room for
            op* o = ep.backlog.front();
            if (!post(ep, o))
                break;
            ep.backlog.pop_front();
        }
    }

    bool has_rma() const override { return false; }
    atl_mr mr_reg(void*, size_t) override {
        CCL_THROW("one-sided writes are not offered by the ofi transport (use the socket transport for CCL_ATL_RMA)");
    }
    void mr_dereg(const atl_mr&) override {}
    void rma_write(int, const void*, size_t, const atl_mr&, uint64_t, atl_req*) override {
        CCL_THROW("one-sided writes are not offered by the ofi transport");
    }

private:
    struct peek_state;
    struct op {
        op_context ctx; // first member: the completion's op_context is the op itself
        atl_req* req;
        bool is_recv;
        const void* sbuf;
        void* rbuf;
        size_t len;
        int peer;
        uint64_t tag;
        peek_state* peek = nullptr;
    };
    struct peek_state {
        op o;
        int state = 0; // 0 pending, 1 message present, 2 no message
        size_t len = 0;
    };
    struct self_msg {
        uint64_t tag;
        std::vector<char> data;
    };
    struct self_posted {
        uint64_t tag;
        void* buf;
        size_t len;
        atl_req* req;
    };
    struct endpoint {
        fid_ep* ep = nullptr;
        fid_cq* cq = nullptr;
        std::vector<fi_addr_t> peer;
        std::mutex mu;
        std::deque<op*> backlog;
        std::map<std::pair<int, uint64_t>, peek_state*> peeks;
        std::list<self_msg> self_unexpected;
        std::list<self_posted> self_recvs;
    };

    bool post(endpoint& ep, op* o) {
        ssize_t rc;
        if (o->is_recv)
            rc = ep.ep->tagged->recv(ep.ep, o->rbuf, o->len, nullptr, ep.peer[o->peer], o->tag, 0, &o->ctx);
        else
            rc = ep.ep->tagged->send(ep.ep, o->sbuf, o->len, nullptr, ep.peer[o->peer], o->tag, &o->ctx);
        if (rc == -E_AGAIN) {
            reap(ep);
            return false;
        }
        OFI_CALL(rc);
        return true;
    }

    void finish(op* o, size_t len, int error) {
        if (o->peek) {
            o->peek->state = error ? 2 : 1;
            o->peek->len = len;
            return; // owned by its peek_state
        }
        if (o->req) {
            if (o->is_recv) {
                o->req->bytes = len;
                bytes_received += len;
            }
            o->req->error = error;
            o->req->done.store(1, std::memory_order_release);
        }
        delete o;
    }

    void reap(endpoint& ep) {
        fi_cq_tagged_entry ent[16];
        for (;;) {
            const ssize_t n = ep.cq->ops->read(ep.cq, ent, 16);
            if (n > 0) {
                for (ssize_t i = 0; i < n; i++)
                    finish((op*)ent[i].op_context, ent[i].len, 0);
                continue;
            }
            if (n == -E_AVAIL) {
                fi_cq_err_entry err{};
                if (ep.cq->ops->readerr(ep.cq, &err, 0) >= 0 && err.op_context) {
                    op* o = (op*)err.op_context;
                    if (o->peek && err.err == E_NOMSG)
                        finish(o, 0, E_NOMSG);
                    else if (err.err == E_TRUNC)
                        finish(o, err.len, 0); // a shorter buffer than the message: what arrived is delivered
                    else {
                        if (err.err != E_CANCELED) {
                            LOG_ERROR("ofi transport: operation with rank ", o->peer, " failed: ",
                                      lib_.strerror ? lib_.strerror(err.err) : "?", " (provider code ", err.prov_errno, ")");
                            peers_lost++;
                        }
                        finish(o, 0, err.err ? err.err : 1);
                    }
                }
                continue;
            }
            break; // -FI_EAGAIN: nothing more
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
        self_msg m{ tag, std::vector<char>((const char*)buf, (const char*)buf + len) };
        ep.self_unexpected.push_back(std::move(m));
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
        ep.self_recvs.push_back(self_posted{ tag, buf, len, req });
    }

    library lib_;
    int rank_, size_;
    std::vector<endpoint> eps_;
    fi_info* info_ = nullptr;
    fid_fabric* fabric_ = nullptr;
    fid_domain* domain_ = nullptr;
    fid_av* av_ = nullptr;
    std::vector<char> same_host_;
    std::string prov_, name_;
};

} // namespace

// Null when libfabric cannot be loaded on SOME rank (the ranks agree through the PMI layer, so that either all
// of them use it or none does); a provider that then fails to come up is an error.
std::shared_ptr<atl_transport> create_ofi_transport(pmi& pm, int ep_count, std::string& why) {
    static library lib;
    static std::mutex mu;
    int ok = 1;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!lib.handle && !load_library(lib, why))
            ok = 0;
    }
    std::vector<int> all(pm.size(), 0);
    pm.allgather(&ok, all.data(), sizeof(int));
    for (int r = 0; r < pm.size(); r++)
        if (!all[r]) {
            if (ok)
                why = "rank " + std::to_string(r) + " could not load libfabric";
            return nullptr;
        }
    return std::make_shared<ofi_transport>(pm, ep_count, lib);
}

} // namespace cclx
