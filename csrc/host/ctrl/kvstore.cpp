#include "ctrl/kvstore.h"

#include <algorithm>
#include <chrono>
#include <stdexcept>

namespace slime {
namespace ctrl {

bool StreamId::parse(const std::string& s, StreamId& out)
{
    if (s.empty()) return false;
    const size_t dash = s.find('-');
    try {
        size_t used = 0;
        out.ms      = std::stoull(s.substr(0, dash), &used);
        if (used != (dash == std::string::npos ? s.size() : dash)) return false;
        out.seq = 0;
        if (dash != std::string::npos) {
            const std::string tail = s.substr(dash + 1);
            out.seq                = std::stoull(tail, &used);
            if (used != tail.size()) return false;
        }
    }
    catch (const std::exception&) {
        return false;
    }
    return true;
}

KvStore::KvStore()
{
    clock_ = [] {
        return static_cast<int64_t>(
            std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
    };
}

void KvStore::set_clock(Clock c)
{
    std::lock_guard<std::mutex> g(mu_);
    clock_ = std::move(c);
}

int64_t KvStore::now_ms() const
{
    return clock_();
}

KvStore::Value* KvStore::find_live(const std::string& key)
{
    auto it = data_.find(key);
    if (it == data_.end()) return nullptr;
    if (it->second.expire_at >= 0 && it->second.expire_at <= clock_()) {
        data_.erase(it);
        return nullptr;
    }
    return &it->second;
}

KvStore::Value& KvStore::get_or_create(const std::string& key, Type t)
{
    Value* v = find_live(key);
    if (v == nullptr) {
        Value nv;
        nv.type = t;
        v       = &data_.emplace(key, std::move(nv)).first->second;
    }
    else if (v->type != t) {
        throw std::runtime_error("WRONGTYPE Operation against a key holding the wrong kind of value");
    }
    return *v;
}

// A live value of kind `t`, nullptr when the key is absent; a key that holds another kind of value is an error for
// reads as well as for writes, as in Redis.
KvStore::Value* KvStore::find_typed(const std::string& key, Type t)
{
    Value* v = find_live(key);
    if (v != nullptr && v->type != t)
        throw std::runtime_error("WRONGTYPE Operation against a key holding the wrong kind of value");
    return v;
}

// ------------------------------------------------------------------ strings / generic
bool KvStore::set(const std::string& key, const std::string& value, int64_t ttl_ms, bool nx)
{
    std::lock_guard<std::mutex> g(mu_);
    if (nx && find_live(key) != nullptr) return false;
    Value v;
    v.type      = Type::String;
    v.str       = value;
    v.expire_at = ttl_ms >= 0 ? clock_() + ttl_ms : -1;
    data_[key]  = std::move(v);
    return true;
}

std::optional<std::string> KvStore::get(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_live(key);
    if (v == nullptr) return std::nullopt;
    if (v->type != Type::String) throw std::runtime_error("WRONGTYPE Operation against a key holding the wrong kind of value");
    return v->str;
}

std::vector<std::optional<std::string>> KvStore::mget(const std::vector<std::string>& keys)
{
    std::lock_guard<std::mutex> g(mu_);
    std::vector<std::optional<std::string>> out;
    for (const auto& k : keys) {
        Value* v = find_live(k);
        if (v != nullptr && v->type == Type::String) out.emplace_back(v->str);
        else out.emplace_back(std::nullopt);
    }
    return out;
}

int64_t KvStore::del(const std::vector<std::string>& keys)
{
    std::lock_guard<std::mutex> g(mu_);
    int64_t n = 0;
    for (const auto& k : keys)
        if (find_live(k) != nullptr) {
            data_.erase(k);
            ++n;
        }
    return n;
}

bool KvStore::exists(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    return find_live(key) != nullptr;
}

bool KvStore::expire(const std::string& key, int64_t ttl_ms)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_live(key);
    if (v == nullptr) return false;
    v->expire_at = clock_() + ttl_ms;
    return true;
}

int64_t KvStore::pttl(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_live(key);
    if (v == nullptr) return -2;
    if (v->expire_at < 0) return -1;
    return std::max<int64_t>(0, v->expire_at - clock_());
}

int64_t KvStore::incr(const std::string& key, int64_t by)
{
    std::lock_guard<std::mutex> g(mu_);
    Value&  v   = get_or_create(key, Type::String);
    int64_t cur = 0;
    if (!v.str.empty()) {
        try {
            size_t used = 0;
            cur         = std::stoll(v.str, &used);
            if (used != v.str.size()) throw std::invalid_argument("x");
        }
        catch (const std::exception&) {
            throw std::runtime_error("ERR value is not an integer or out of range");
        }
    }
    cur += by;
    v.str = std::to_string(cur);
    return cur;
}

bool KvStore::glob_match(const std::string& pattern, const std::string& text)
{
    // iterative matcher with backtracking over the last '*'
    size_t p = 0, t = 0, star = std::string::npos, mark = 0;
    auto   class_match = [&](size_t& pi, char c) -> bool {
        // pattern[pi] == '['
        size_t i = pi + 1;
        bool   neg = false, ok = false;
        if (i < pattern.size() && pattern[i] == '^') {
            neg = true;
            ++i;
        }
        while (i < pattern.size() && pattern[i] != ']') {
            if (i + 2 < pattern.size() && pattern[i + 1] == '-' && pattern[i + 2] != ']') {
                if (c >= pattern[i] && c <= pattern[i + 2]) ok = true;
                i += 3;
            }
            else {
                if (pattern[i] == '\\' && i + 1 < pattern.size()) ++i;
                if (pattern[i] == c) ok = true;
                ++i;
            }
        }
        pi = i < pattern.size() ? i + 1 : i;
        return neg ? !ok : ok;
    };
    while (t < text.size()) {
        if (p < pattern.size() && pattern[p] == '*') {
            star = p++;
            mark = t;
            continue;
        }
        bool   matched = false;
        size_t np      = p;
        if (p < pattern.size()) {
            if (pattern[p] == '?') {
                matched = true;
                np      = p + 1;
            }
            else if (pattern[p] == '[') {
                size_t pi = p;
                matched   = class_match(pi, text[t]);
                np        = pi;
            }
            else {
                size_t pi = p;
                if (pattern[pi] == '\\' && pi + 1 < pattern.size()) ++pi;
                matched = pattern[pi] == text[t];
                np      = pi + 1;
            }
        }
        if (matched) {
            p = np;
            ++t;
        }
        else if (star != std::string::npos) {
            p = star + 1;
            t = ++mark;
        }
        else {
            return false;
        }
    }
    while (p < pattern.size() && pattern[p] == '*') ++p;
    return p == pattern.size();
}

std::vector<std::string> KvStore::keys(const std::string& pattern)
{
    std::lock_guard<std::mutex> g(mu_);
    std::vector<std::string> out;
    const int64_t now = clock_();
    for (const auto& kv : data_) {
        if (kv.second.expire_at >= 0 && kv.second.expire_at <= now) continue;
        if (glob_match(pattern, kv.first)) out.push_back(kv.first);
    }
    return out;
}

std::pair<uint64_t, std::vector<std::string>> KvStore::scan(uint64_t cursor, const std::string& pattern, size_t count)
{
    // the cursor is the rank of the next key in sorted order; good enough for a single-writer control plane
    std::lock_guard<std::mutex> g(mu_);
    std::vector<std::string> out;
    const int64_t now  = clock_();
    uint64_t      rank = 0;
    if (count == 0) count = 10;
    size_t visited = 0;
    for (auto it = data_.begin(); it != data_.end(); ++it, ++rank) {
        if (rank < cursor) continue;
        if (visited >= count) return {rank, out};
        ++visited;
        if (it->second.expire_at >= 0 && it->second.expire_at <= now) continue;
        if (glob_match(pattern, it->first)) out.push_back(it->first);
    }
    return {0, out};
}

std::string KvStore::type_of(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_live(key);
    if (v == nullptr) return "none";
    switch (v->type) {
        case Type::String: return "string";
        case Type::Hash: return "hash";
        case Type::List: return "list";
        case Type::Stream: return "stream";
    }
    return "none";
}

void KvStore::flush_all()
{
    std::lock_guard<std::mutex> g(mu_);
    data_.clear();
}

size_t KvStore::size()
{
    std::lock_guard<std::mutex> g(mu_);
    return data_.size();
}

// ------------------------------------------------------------------ hashes
int64_t KvStore::hset(const std::string& key, const std::vector<std::pair<std::string, std::string>>& fields)
{
    std::lock_guard<std::mutex> g(mu_);
    Value&  v = get_or_create(key, Type::Hash);
    int64_t added = 0;
    for (const auto& f : fields) {
        added += v.hash.count(f.first) ? 0 : 1;
        v.hash[f.first] = f.second;
    }
    return added;
}

std::optional<std::string> KvStore::hget(const std::string& key, const std::string& field)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::Hash);
    if (v == nullptr) return std::nullopt;
    auto it = v->hash.find(field);
    if (it == v->hash.end()) return std::nullopt;
    return it->second;
}

std::vector<std::pair<std::string, std::string>> KvStore::hgetall(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::Hash);
    if (v == nullptr) return {};
    return {v->hash.begin(), v->hash.end()};
}

int64_t KvStore::hdel(const std::string& key, const std::vector<std::string>& fields)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::Hash);
    if (v == nullptr) return 0;
    int64_t n = 0;
    for (const auto& f : fields) n += static_cast<int64_t>(v->hash.erase(f));
    if (v->hash.empty()) data_.erase(key);
    return n;
}

// ------------------------------------------------------------------ lists
int64_t KvStore::lpush(const std::string& key, const std::vector<std::string>& values)
{
    int64_t n;
    {
        std::lock_guard<std::mutex> g(mu_);
        Value& v = get_or_create(key, Type::List);
        for (const auto& s : values) v.list.push_front(s);
        n = static_cast<int64_t>(v.list.size());
    }
    cv_.notify_all();
    return n;
}

int64_t KvStore::rpush(const std::string& key, const std::vector<std::string>& values)
{
    int64_t n;
    {
        std::lock_guard<std::mutex> g(mu_);
        Value& v = get_or_create(key, Type::List);
        for (const auto& s : values) v.list.push_back(s);
        n = static_cast<int64_t>(v.list.size());
    }
    cv_.notify_all();
    return n;
}

std::optional<std::string> KvStore::lpop(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::List);
    if (v == nullptr || v->list.empty()) return std::nullopt;
    std::string s = std::move(v->list.front());
    v->list.pop_front();
    if (v->list.empty()) data_.erase(key);
    return s;
}

std::optional<std::string> KvStore::rpop(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::List);
    if (v == nullptr || v->list.empty()) return std::nullopt;
    std::string s = std::move(v->list.back());
    v->list.pop_back();
    if (v->list.empty()) data_.erase(key);
    return s;
}

int64_t KvStore::llen(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::List);
    return v == nullptr ? 0 : static_cast<int64_t>(v->list.size());
}

std::vector<std::string> KvStore::lrange(const std::string& key, int64_t start, int64_t stop)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::List);
    if (v == nullptr) return {};
    const int64_t n = static_cast<int64_t>(v->list.size());
    if (start < 0) start = std::max<int64_t>(0, n + start);
    if (stop < 0) stop = n + stop;
    stop = std::min(stop, n - 1);
    std::vector<std::string> out;
    for (int64_t i = start; i <= stop; ++i) out.push_back(v->list[static_cast<size_t>(i)]);
    return out;
}

std::optional<std::pair<std::string, std::string>> KvStore::blpop(const std::vector<std::string>& keys, int64_t timeout_ms)
{
    std::unique_lock<std::mutex> g(mu_);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    while (true) {
        for (const auto& k : keys) {
            Value* v = find_live(k);
            if (v != nullptr && v->type == Type::List && !v->list.empty()) {
                std::string s = std::move(v->list.front());
                v->list.pop_front();
                if (v->list.empty()) data_.erase(k);
                return std::make_pair(k, std::move(s));
            }
        }
        if (interrupted_.load()) return std::nullopt;
        if (timeout_ms <= 0) {
            cv_.wait_for(g, std::chrono::milliseconds(200));  // periodic wake-up so interrupt() is seen
        }
        else if (cv_.wait_until(g, deadline) == std::cv_status::timeout) {
            return std::nullopt;
        }
    }
}

// ------------------------------------------------------------------ streams
std::string KvStore::xadd(const std::string& key, const std::string& id,
                          const std::vector<std::pair<std::string, std::string>>& fields, size_t maxlen)
{
    std::string out;
    {
        std::lock_guard<std::mutex> g(mu_);
        Value&   v = get_or_create(key, Type::Stream);
        StreamId nid;
        if (id == "*") {
            nid.ms = static_cast<uint64_t>(clock_());
            if (nid.ms <= v.last_id.ms) {
                nid.ms  = v.last_id.ms;
                nid.seq = v.last_id.seq + 1;
            }
        }
        else {
            if (!StreamId::parse(id, nid)) return "";
            if (!(v.last_id < nid)) return "";
        }
        StreamEntry e;
        e.id     = nid;
        e.fields = fields;
        v.stream.push_back(std::move(e));
        v.last_id = nid;
        if (maxlen > 0 && v.stream.size() > maxlen) v.stream.erase(v.stream.begin(), v.stream.end() - static_cast<long>(maxlen));
        out = nid.str();
    }
    cv_.notify_all();
    return out;
}

int64_t KvStore::xlen(const std::string& key)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::Stream);
    return v == nullptr ? 0 : static_cast<int64_t>(v->stream.size());
}

std::vector<std::pair<std::string, std::vector<StreamEntry>>>
KvStore::xread(const std::vector<std::pair<std::string, std::string>>& keys_ids, size_t count, int64_t block_ms)
{
    std::unique_lock<std::mutex> g(mu_);
    // resolve "$" once, at call time
    std::vector<StreamId> after(keys_ids.size());
    for (size_t i = 0; i < keys_ids.size(); ++i) {
        if (keys_ids[i].second == "$") {
            Value* v = find_live(keys_ids[i].first);
            after[i] = (v != nullptr && v->type == Type::Stream) ? v->last_id : StreamId{};
        }
        else if (!StreamId::parse(keys_ids[i].second, after[i])) {
            throw std::runtime_error("ERR Invalid stream ID specified as stream command argument");
        }
    }
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(block_ms > 0 ? block_ms : 0);
    while (true) {
        std::vector<std::pair<std::string, std::vector<StreamEntry>>> out;
        for (size_t i = 0; i < keys_ids.size(); ++i) {
            Value* v = find_live(keys_ids[i].first);
            if (v == nullptr || v->type != Type::Stream) continue;
            std::vector<StreamEntry> got;
            auto it = std::upper_bound(v->stream.begin(), v->stream.end(), after[i],
                                       [](const StreamId& a, const StreamEntry& e) { return a < e.id; });
            for (; it != v->stream.end() && (count == 0 || got.size() < count); ++it) got.push_back(*it);
            if (!got.empty()) out.emplace_back(keys_ids[i].first, std::move(got));
        }
        if (!out.empty() || block_ms < 0 || interrupted_.load()) return out;
        if (block_ms == 0) {
            cv_.wait_for(g, std::chrono::milliseconds(200));
        }
        else if (cv_.wait_until(g, deadline) == std::cv_status::timeout) {
            return out;
        }
    }
}

std::vector<StreamEntry> KvStore::xrange(const std::string& key, const std::string& start, const std::string& end, size_t count)
{
    std::lock_guard<std::mutex> g(mu_);
    Value* v = find_typed(key, Type::Stream);
    if (v == nullptr) return {};
    StreamId lo{0, 0}, hi{UINT64_MAX, UINT64_MAX};
    if (start != "-" && !StreamId::parse(start, lo)) throw std::runtime_error("ERR Invalid stream ID");
    if (end != "+" && !StreamId::parse(end, hi)) throw std::runtime_error("ERR Invalid stream ID");
    std::vector<StreamEntry> out;
    for (const auto& e : v->stream) {
        if (e.id < lo || hi < e.id) continue;
        out.push_back(e);
        if (count && out.size() >= count) break;
    }
    return out;
}

// ------------------------------------------------------------------ publish / subscribe
int64_t KvStore::publish(const std::string& channel, const std::string& message)
{
    std::vector<Subscriber> targets;
    {
        std::lock_guard<std::mutex> g(sub_mu_);
        for (const auto& kv : subs_)
            if (kv.second.first == channel || glob_match(kv.second.first, channel)) targets.push_back(kv.second.second);
    }
    for (auto& fn : targets) fn(channel, message);
    return static_cast<int64_t>(targets.size());
}

uint64_t KvStore::subscribe(const std::string& channel, Subscriber fn)
{
    std::lock_guard<std::mutex> g(sub_mu_);
    const uint64_t t = next_token_++;
    subs_[t]         = {channel, std::move(fn)};
    return t;
}

void KvStore::unsubscribe(uint64_t token)
{
    std::lock_guard<std::mutex> g(sub_mu_);
    subs_.erase(token);
}

void KvStore::interrupt()
{
    interrupted_.store(true);
    cv_.notify_all();
}

}  // namespace ctrl
}  // namespace slime
