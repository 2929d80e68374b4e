#include "ctrl/obs_view.h"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <netdb.h>
#include <stdexcept>
#include <sys/socket.h>
#include <unistd.h>

namespace slime {
namespace ctrl {

namespace {

// Minimal blocking RESP2 client: enough for SCAN and MGET.
class Resp {
public:
    Resp(const std::string& address)
    {
        std::string a = address;
        const size_t scheme = a.find("://");
        if (scheme != std::string::npos) a = a.substr(scheme + 3);
        const size_t slash = a.find('/');
        if (slash != std::string::npos) a.resize(slash);
        const size_t colon = a.rfind(':');
        const std::string host = colon == std::string::npos ? a : a.substr(0, colon);
        const std::string port = colon == std::string::npos ? "6379" : a.substr(colon + 1);
        addrinfo hints{}, *res = nullptr;
        hints.ai_family   = AF_INET;
        hints.ai_socktype = SOCK_STREAM;
        if (getaddrinfo(host.empty() ? "127.0.0.1" : host.c_str(), port.c_str(), &hints, &res) != 0 || !res)
            throw std::runtime_error("cannot resolve " + address);
        fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
        const bool ok = fd_ >= 0 && ::connect(fd_, res->ai_addr, res->ai_addrlen) == 0;
        freeaddrinfo(res);
        if (!ok) throw std::runtime_error("cannot connect to the store at " + address);
    }
    ~Resp()
    {
        if (fd_ >= 0) ::close(fd_);
    }
    Json command(const std::vector<std::string>& argv)
    {
        std::string out = "*" + std::to_string(argv.size()) + "\r\n";
        for (const auto& a : argv) out += "$" + std::to_string(a.size()) + "\r\n" + a + "\r\n";
        if (::send(fd_, out.data(), out.size(), MSG_NOSIGNAL) != static_cast<ssize_t>(out.size())) throw std::runtime_error("store write failed");
        return reply();
    }

private:
    void fill()
    {
        char    tmp[16384];
        ssize_t n = ::recv(fd_, tmp, sizeof(tmp), 0);
        if (n <= 0) throw std::runtime_error("store connection closed");
        buf_.append(tmp, static_cast<size_t>(n));
    }
    std::string line()
    {
        size_t nl;
        while ((nl = buf_.find("\r\n", pos_)) == std::string::npos) fill();
        std::string s = buf_.substr(pos_, nl - pos_);
        pos_          = nl + 2;
        return s;
    }
    Json reply()
    {
        const std::string l = line();
        switch (l[0]) {
            case '+': return Json(l.substr(1));
            case '-': throw std::runtime_error("store error: " + l.substr(1));
            case ':': return Json(static_cast<long long>(std::strtoll(l.c_str() + 1, nullptr, 10)));
            case '$': {
                const long n = std::strtol(l.c_str() + 1, nullptr, 10);
                if (n < 0) return Json();
                while (buf_.size() - pos_ < static_cast<size_t>(n) + 2) fill();
                Json v(buf_.substr(pos_, static_cast<size_t>(n)));
                pos_ += static_cast<size_t>(n) + 2;
                return v;
            }
            case '*': {
                const long n = std::strtol(l.c_str() + 1, nullptr, 10);
                Json       arr = Json::array();
                for (long i = 0; i < n; ++i) arr.push_back(reply());
                return arr;
            }
            default: throw std::runtime_error("bad store reply");
        }
    }
    int         fd_ = -1;
    std::string buf_;
    size_t      pos_ = 0;
};

std::string table(const std::vector<std::string>& header, const std::vector<std::vector<std::string>>& rows)
{
    std::vector<size_t> w(header.size());
    for (size_t i = 0; i < header.size(); ++i) w[i] = header[i].size();
    for (const auto& r : rows)
        for (size_t i = 0; i < r.size() && i < w.size(); ++i) w[i] = std::max(w[i], r[i].size());
    auto line = [&](const std::vector<std::string>& r) {
        std::string s;
        for (size_t i = 0; i < w.size(); ++i) {
            const std::string c = i < r.size() ? r[i] : "";
            s += c + std::string(w[i] - c.size() + 2, ' ');
        }
        while (!s.empty() && s.back() == ' ') s.pop_back();
        return s + "\n";
    };
    std::string out = line(header);
    std::vector<std::string> rule;
    for (size_t i = 0; i < w.size(); ++i) rule.push_back(std::string(w[i], '-'));
    out += line(rule);
    for (const auto& r : rows) out += line(r);
    return out;
}

std::string num(const Json& j)
{
    return j.is_null() ? "-" : std::to_string(j.as_int());
}

}  // namespace

std::string snapshot_state(const Json& snap, int64_t now_ms, int64_t stale_ms)
{
    if (snap["status"].string_or("") == "stopped") return "stopped";
    const int64_t at = snap["reported_at_ms"].as_int();
    return (at == 0 || now_ms - at > stale_ms) ? "stale" : "alive";
}

std::string human_bps(double v)
{
    const char* unit[] = {"bps", "Kbps", "Mbps", "Gbps", "Tbps"};
    int         u = 0;
    while (v >= 1000.0 && u < 4) {
        v /= 1000.0;
        ++u;
    }
    char buf[32];
    snprintf(buf, sizeof(buf), u == 0 ? "%.0f %s" : "%.2f %s", v, unit[u]);
    return buf;
}

std::string human_bytes(double v)
{
    const char* unit[] = {"B", "KiB", "MiB", "GiB", "TiB"};
    int         u = 0;
    while (v >= 1024.0 && u < 4) {
        v /= 1024.0;
        ++u;
    }
    char buf[32];
    snprintf(buf, sizeof(buf), u == 0 ? "%.0f %s" : "%.2f %s", v, unit[u]);
    return buf;
}

std::vector<PeerSnapshot> fetch_snapshots(const std::string& address, const std::string& scope, int64_t stale_ms)
{
    Resp              r(address);
    const std::string prefix = (scope.empty() ? "" : scope + ":") + "obs:peer:";
    std::vector<std::string> keys;
    std::string cursor = "0";
    do {
        Json res = r.command({"SCAN", cursor, "MATCH", prefix + "*", "COUNT", "200"});
        cursor   = res[0].as_string();
        for (const auto& k : res[1].items()) keys.push_back(k.as_string());
    } while (cursor != "0");
    std::sort(keys.begin(), keys.end());
    std::vector<PeerSnapshot> out;
    if (keys.empty()) return out;
    std::vector<std::string> cmd{"MGET"};
    cmd.insert(cmd.end(), keys.begin(), keys.end());
    Json vals = r.command(cmd);
    const int64_t now = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
    for (size_t i = 0; i < keys.size(); ++i) {
        Json snap;
        if (!vals[i].is_string() || !Json::try_parse(vals[i].as_string(), snap)) continue;
        PeerSnapshot p;
        p.alias  = keys[i].substr(prefix.size());
        p.state  = snapshot_state(snap, now, stale_ms);
        p.age_ms = now - snap["reported_at_ms"].as_int();
        p.data   = snap;
        out.push_back(std::move(p));
    }
    return out;
}

std::string render_obs_view(const std::vector<PeerSnapshot>& peers, const std::string& view, bool as_json)
{
    if (as_json) {
        Json arr = Json::array();
        for (const auto& p : peers) {
            Json e     = p.data;
            e["state"] = p.state;
            e["age_ms"] = static_cast<long long>(p.age_ms);
            arr.push_back(e);
        }
        return arr.dump(2) + "\n";
    }
    if (view == "status") {
        size_t alive = 0, stale = 0, stopped = 0;
        double bw = 0;
        for (const auto& p : peers) {
            alive += p.state == "alive";
            stale += p.state == "stale";
            stopped += p.state == "stopped";
            if (p.state == "alive") bw += p.data["ewma_bandwidth_bps"].as_double();
        }
        char buf[256];
        snprintf(buf, sizeof(buf), "peers: %zu alive, %zu stale, %zu stopped; aggregate bandwidth %s\n", alive, stale, stopped, human_bps(bw).c_str());
        return buf;
    }
    if (view == "peers") {
        std::vector<std::vector<std::string>> rows;
        for (const auto& p : peers) {
            const Json& s = p.data["summary"];
            rows.push_back({p.alias, p.state, p.data["host"].string_or("-"), num(p.data["pid"]), std::to_string(p.age_ms / 1000) + "s",
                            num(s["pending_ops"]), human_bytes(s["completed_bytes_total"].as_double()), num(s["error_total"]),
                            num(s["mr_count"]), human_bps(p.data["ewma_bandwidth_bps"].as_double())});
        }
        return table({"PEER", "STATE", "HOST", "PID", "AGE", "PENDING", "COMPLETED", "ERRORS", "MRS", "BANDWIDTH"}, rows);
    }
    if (view == "nics") {
        std::vector<std::vector<std::string>> rows;
        for (const auto& p : peers)
            for (const auto& n : p.data["nics"].items())
                rows.push_back({p.alias, n["nic"].string_or("-"), n["kind"].string_or("rdma"), num(n["pending_ops"]),
                                human_bytes(n["completed_bytes_total"].as_double()), num(n["post_failures_total"]), num(n["cq_errors_total"]),
                                human_bps(n["ewma_bandwidth_bps"].as_double())});
        return table({"PEER", "LINK", "KIND", "PENDING", "COMPLETED", "POST_FAIL", "CQ_ERR", "BANDWIDTH"}, rows);
    }
    if (view == "links") {
        std::vector<std::vector<std::string>> rows;
        for (const auto& p : peers)
            for (const auto& c : p.data["connections"].items())
                rows.push_back({p.alias, c["peer"].string_or("-"), c["local_nic"].string_or("-"), c["remote_nic"].string_or("-"),
                                c["state"].string_or("-"), c["conn_id"].string_or("-")});
        return table({"PEER", "REMOTE", "LOCAL_LINK", "REMOTE_LINK", "STATE", "CONNECTION"}, rows);
    }
    return "unknown view '" + view + "' (status | peers | nics | links)\n";
}

int obs_view_main(const std::string& address, const std::string& scope, const std::string& view, int64_t stale_ms, bool as_json)
{
    try {
        const auto peers = fetch_snapshots(address, scope, stale_ms);
        fputs(render_obs_view(peers, view, as_json).c_str(), stdout);
        return 0;
    }
    catch (const std::exception& e) {
        fprintf(stderr, "nanoctrl obs: %s\n", e.what());
        return 1;
    }
}

}  // namespace ctrl
}  // namespace slime
