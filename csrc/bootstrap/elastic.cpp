#include "bootstrap/elastic.hpp"

#include <algorithm>
#include <chrono>
#include <sstream>

#include "core/log.hpp"

namespace cclx {

namespace {
long long now_ms() {
    using namespace std::chrono;
    return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}
std::string to_s(const kvs::bytes& b) {
    return std::string(b.begin(), b.end());
}
kvs::bytes to_b(const std::string& s) {
    return kvs::bytes(s.begin(), s.end());
}
const char* const POD = "elastic/pods/";
const char* const HB = "elastic/hb/";
} // namespace

scoped_kvs::scoped_kvs(std::shared_ptr<kvs::ikvs> base, std::string prefix)
        : base_(std::move(base)), prefix_(std::move(prefix)) {
    addr_ = kvs::address::from_string(base_->get_address().str() + "|" + prefix_);
}

elastic_group::elastic_group(std::shared_ptr<kvs::internal_kvs> store, std::string pod_id, int heartbeat_ms,
                             int dead_after_ms)
        : store_(std::move(store)), id_(std::move(pod_id)), hb_ms_(heartbeat_ms), dead_ms_(dead_after_ms) {
    CCL_THROW_IF_NOT(!id_.empty() && id_.find('/') == std::string::npos && id_.find(',') == std::string::npos,
                     "pod id must be non-empty and free of '/' and ','");
    CCL_THROW_IF_NOT(hb_ms_ > 0 && dead_ms_ > 2 * hb_ms_, "dead_after_ms must be more than two heartbeats");
}

elastic_group::~elastic_group() {
    try {
        leave();
    }
    catch (...) {
    }
}

void elastic_group::beat_loop() {
    while (!stop_.load()) {
        try {
            store_->raw().add(HB + id_, 1);
        }
        catch (const std::exception&) {
            return; // the store is gone: nothing left to report to
        }
        for (int waited = 0; waited < hb_ms_ && !stop_.load(); waited += 10)
            std::this_thread::sleep_for(std::chrono::milliseconds(std::min(10, hb_ms_)));
    }
}

void elastic_group::leave() {
    if (!registered_)
        return;
    stop_.store(true);
    if (beat_.joinable())
        beat_.join();
    store_->raw().del(POD + id_);
    store_->raw().del(HB + id_);
    registered_ = false;
}

// registered pods whose heartbeat moved within dead_after_ms; a pod seen for the first time gets
// `settle_ms` to prove itself before it counts as dead
std::vector<std::string> elastic_group::live_pods(int settle_ms) {
    std::vector<std::string> out;
    const long long t = now_ms();
    auto pods = store_->raw().list(POD);
    std::map<std::string, seen> next;
    for (auto& kv : pods) {
        const std::string id = kv.first.substr(std::string(POD).size());
        ticket_[id] = std::atoll(to_s(kv.second).c_str());
        kvs::bytes b;
        long long v = -1;
        if (store_->raw().try_get(HB + id, b))
            v = std::atoll(to_s(b).c_str());
        seen s = seen_.count(id) ? seen_[id] : seen{ -2, t + settle_ms - dead_ms_ };
        if (v != s.value) {
            s.value = v;
            s.changed_at = t;
        }
        next[id] = s;
        if (id == id_ || t - s.changed_at <= dead_ms_)
            out.push_back(id);
    }
    seen_.swap(next);
    std::sort(out.begin(), out.end(), [&](const std::string& a, const std::string& b) {
        return ticket_[a] != ticket_[b] ? ticket_[a] < ticket_[b] : a < b;
    });
    return out;
}

bool elastic_group::changed() {
    CCL_THROW_IF_NOT(registered_, "form() has not been called");
    return live_pods(dead_ms_) != view_.members;
}

elastic_group::view elastic_group::form(int timeout_ms) {
    if (!registered_) {
        const long long ticket = store_->raw().add("elastic/ticket", 1);
        store_->raw().set(POD + id_, std::to_string(ticket));
        store_->raw().add(HB + id_, 1);
        stop_.store(false);
        beat_ = std::thread([this] { beat_loop(); });
        registered_ = true;
    }
    const long long deadline = now_ms() + timeout_ms;
    // Agreement in two phases per generation g.  (1) Every live pod publishes its member list under
    // elastic/view/<g>/<id> and waits until all listed pods published the same list.  (2) Each then writes
    // elastic/commit/<g>/<id> and returns the view only when all n commits are there.  A pod that wants to
    // withdraw its list (it saw a different list, or the live set moved) first looks for commits of g: once any
    // exists, everybody had published this very list, so it commits too instead of withdrawing.  A generation
    // that failed is never tried again (its keys are stale): the failure raises elastic/floor, and every pod
    // starts its next attempt at max(adopted + 1, floor), so the pods meet again at one number.
    auto read_num = [&](const char* key) -> uint64_t {
        kvs::bytes b;
        return store_->raw().try_get(key, b) ? (uint64_t)std::atoll(to_s(b).c_str()) : 0;
    };
    for (;;) {
        CCL_THROW_IF_NOT(now_ms() < deadline, "elastic group: no agreement on a member list within ", timeout_ms, " ms");
        const uint64_t g = std::max<uint64_t>({ read_num("elastic/adopted") + 1, read_num("elastic/floor"),
                                                view_.generation + 1, floor_ });
        std::vector<std::string> mine = live_pods(dead_ms_);
        const size_t n = mine.size();
        resize_action act = resize_fn_ ? resize_fn_(n) : (n >= min_size_ ? resize_action::run : resize_action::wait);
        CCL_THROW_IF_NOT(act != resize_action::finalize, "elastic group: the resize function asked to finalize at size ", n);
        if (act == resize_action::wait) {
            std::this_thread::sleep_for(std::chrono::milliseconds(hb_ms_));
            continue;
        }
        std::string list;
        for (auto& m : mine)
            list += (list.empty() ? "" : ",") + m;
        const std::string base = "elastic/view/" + std::to_string(g) + "/";
        const std::string cbase = "elastic/commit/" + std::to_string(g) + "/";
        store_->raw().set(base + id_, list);
        if (window_hook_)
            window_hook_(g); // tests: something happens between publishing and agreeing
        // phase 1: every listed member published the same list (or somebody disagrees / the set moves)
        bool agreed = false;
        const long long round_end = std::min<long long>(deadline, now_ms() + 4LL * dead_ms_);
        while (now_ms() < round_end) {
            size_t same = 0;
            bool differ = false;
            for (auto& m : mine) {
                kvs::bytes b;
                if (!store_->raw().try_get(base + m, b))
                    continue;
                if (to_s(b) == list)
                    same++;
                else
                    differ = true;
            }
            if (same == n) {
                agreed = true;
                break;
            }
            if (differ || live_pods(dead_ms_) != mine)
                break;
            std::this_thread::sleep_for(std::chrono::milliseconds(std::max(1, hb_ms_ / 4)));
        }
        if (!agreed && !store_->raw().list(cbase).empty())
            agreed = true; // somebody saw all n lists equal, mine among them: the list stands
        bool committed = false;
        if (agreed) {
            // phase 2: all n commit, or nobody adopts
            store_->raw().set(cbase + id_, "1");
            // no round limit here: the others have published this list and will commit unless they withdrew in
            // the moment before my commit became visible, or died
            while (now_ms() < deadline) {
                size_t have = 0;
                bool lost = false;
                std::vector<std::string> live = live_pods(dead_ms_);
                for (auto& m : mine) {
                    kvs::bytes b;
                    if (store_->raw().try_get(cbase + m, b))
                        have++;
                    else if (!store_->raw().try_get(base + m, b) || to_s(b) != list)
                        lost = true; // it took its list back before it saw a commit: it will not commit
                    else if (std::find(live.begin(), live.end(), m) == live.end())
                        lost = true; // it died in between
                }
                if (have == n) {
                    committed = true;
                    break;
                }
                if (lost)
                    break;
                std::this_thread::sleep_for(std::chrono::milliseconds(std::max(1, hb_ms_ / 4)));
            }
        }
        if (!committed) {
            if (!agreed)
                store_->raw().del(base + id_); // tells a pod that already waits for commits not to wait for mine
            floor_ = g + 1;
            if (read_num("elastic/floor") < floor_)
                store_->raw().set("elastic/floor", std::to_string(floor_));
            std::this_thread::sleep_for(std::chrono::milliseconds(hb_ms_));
            continue;
        }
        if (read_num("elastic/adopted") < g)
            store_->raw().set("elastic/adopted", std::to_string(g));
        view_.generation = g;
        view_.members = mine;
        view_.size = (int)n;
        view_.rank = (int)(std::find(mine.begin(), mine.end(), id_) - mine.begin());
        LOG_INFO("elastic group: generation ", g, ", rank ", view_.rank, " of ", n);
        return view_;
    }
}

std::shared_ptr<kvs::ikvs> elastic_group::generation_store() {
    CCL_THROW_IF_NOT(view_.generation > 0, "form() has not been called");
    return std::make_shared<scoped_kvs>(store_, "elastic/g" + std::to_string(view_.generation) + "/");
}

} // namespace cclx
