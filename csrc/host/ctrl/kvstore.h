// In-memory key-value store with the Redis semantics the control plane relies on:
// strings, hashes, lists and streams, key expiry with an injectable clock, blocking
// list pops and stream reads, glob-pattern scans, counters, and publish / subscribe.
// It backs the embedded NanoCtrl (the reference keeps this state in an external Redis,
// NanoCtrl/README.md:321-337 in the reference) and is served to other processes through
// the RESP2 front-end, so PeerAgents use the same key schema either way.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <utility>
#include <vector>

namespace slime {
namespace ctrl {

struct StreamId {
    uint64_t ms = 0, seq = 0;
    bool operator<(const StreamId& o) const { return ms < o.ms || (ms == o.ms && seq < o.seq); }
    bool operator==(const StreamId& o) const { return ms == o.ms && seq == o.seq; }
    std::string str() const { return std::to_string(ms) + "-" + std::to_string(seq); }
    static bool parse(const std::string& s, StreamId& out);
};

struct StreamEntry {
    StreamId                                         id;
    std::vector<std::pair<std::string, std::string>> fields;
};

class KvStore {
public:
    using Clock = std::function<int64_t()>;  // milliseconds since the epoch

    KvStore();
    void set_clock(Clock c);  // tests drive expiry with a fake clock
    int64_t now_ms() const;

    // ---- strings / generic
    bool                       set(const std::string& key, const std::string& value, int64_t ttl_ms = -1, bool nx = false);
    std::optional<std::string> get(const std::string& key);
    std::vector<std::optional<std::string>> mget(const std::vector<std::string>& keys);
    int64_t del(const std::vector<std::string>& keys);
    bool    exists(const std::string& key);
    bool    expire(const std::string& key, int64_t ttl_ms);
    int64_t pttl(const std::string& key);  // -2 missing, -1 no expiry
    int64_t incr(const std::string& key, int64_t by = 1);
    std::vector<std::string> keys(const std::string& pattern);
    // cursor-based scan: returns the next cursor (0 = done) and up to `count` matching keys
    std::pair<uint64_t, std::vector<std::string>> scan(uint64_t cursor, const std::string& pattern, size_t count);
    std::string type_of(const std::string& key);
    void        flush_all();
    size_t      size();

    // ---- hashes
    int64_t hset(const std::string& key, const std::vector<std::pair<std::string, std::string>>& fields);
    std::optional<std::string> hget(const std::string& key, const std::string& field);
    std::vector<std::pair<std::string, std::string>> hgetall(const std::string& key);
    int64_t hdel(const std::string& key, const std::vector<std::string>& fields);

    // ---- lists
    int64_t lpush(const std::string& key, const std::vector<std::string>& values);
    int64_t rpush(const std::string& key, const std::vector<std::string>& values);
    std::optional<std::string> lpop(const std::string& key);
    std::optional<std::string> rpop(const std::string& key);
    int64_t llen(const std::string& key);
    std::vector<std::string> lrange(const std::string& key, int64_t start, int64_t stop);
    // Blocks up to timeout_ms (0 = for ever) for an element of any listed key: (key, value).
    std::optional<std::pair<std::string, std::string>> blpop(const std::vector<std::string>& keys, int64_t timeout_ms);

    // ---- streams
    // id "*" picks the next id; maxlen > 0 trims the oldest entries. Returns the id or "" on a bad id.
    std::string xadd(const std::string& key, const std::string& id, const std::vector<std::pair<std::string, std::string>>& fields,
                     size_t maxlen = 0);
    int64_t xlen(const std::string& key);
    // Entries with id > after for every (key, after) pair; "$" means "only new entries". block_ms < 0:
    // do not block; 0: block for ever; > 0: block that long.
    std::vector<std::pair<std::string, std::vector<StreamEntry>>> xread(const std::vector<std::pair<std::string, std::string>>& keys_ids,
                                                                        size_t count, int64_t block_ms);
    std::vector<StreamEntry> xrange(const std::string& key, const std::string& start, const std::string& end, size_t count);

    // ---- publish / subscribe
    using Subscriber = std::function<void(const std::string& channel, const std::string& message)>;
    int64_t publish(const std::string& channel, const std::string& message);
    uint64_t subscribe(const std::string& channel, Subscriber fn);  // returns a token
    void     unsubscribe(uint64_t token);

    // Wakes every blocked caller (used at shutdown); they return empty-handed.
    void interrupt();

    static bool glob_match(const std::string& pattern, const std::string& text);

private:
    enum class Type { String, Hash, List, Stream };
    struct Value {
        Type                               type = Type::String;
        std::string                        str;
        std::map<std::string, std::string> hash;
        std::deque<std::string>            list;
        std::vector<StreamEntry>           stream;
        StreamId                           last_id;
        int64_t                            expire_at = -1;
    };
    Value* find_live(const std::string& key);  // expires lazily; caller holds mu_
    Value& get_or_create(const std::string& key, Type t);
    Value* find_typed(const std::string& key, Type t);

    std::mutex                   mu_;
    std::condition_variable      cv_;
    std::map<std::string, Value> data_;
    Clock                        clock_;
    std::atomic<bool>            interrupted_{false};
    std::mutex                   sub_mu_;
    std::map<uint64_t, std::pair<std::string, Subscriber>> subs_;
    uint64_t                     next_token_ = 1;
};

}  // namespace ctrl
}  // namespace slime
