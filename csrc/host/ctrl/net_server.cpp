#include "ctrl/net_server.h"

#include <algorithm>
#include <arpa/inet.h>
#include <cctype>
#include <cerrno>
#include <cstring>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdexcept>
#include <sys/socket.h>
#include <unistd.h>

namespace slime {
namespace ctrl {

namespace {

bool write_all(int fd, const std::string& s)
{
    const char* p = s.data();
    size_t      n = s.size();
    while (n > 0) {
        ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += w;
        n -= static_cast<size_t>(w);
    }
    return true;
}

// Buffered reader over a socket.
struct Reader {
    int         fd;
    std::string buf;
    size_t      pos = 0;

    bool fill()
    {
        if (pos > 0 && pos == buf.size()) {
            buf.clear();
            pos = 0;
        }
        char    tmp[16384];
        ssize_t r;
        do {
            r = ::recv(fd, tmp, sizeof(tmp), 0);
        } while (r < 0 && errno == EINTR);
        if (r <= 0) return false;
        buf.append(tmp, static_cast<size_t>(r));
        return true;
    }
    // Reads up to and including "\r\n" (or "\n"); returns the line without the terminator.
    bool line(std::string& out)
    {
        while (true) {
            const size_t nl = buf.find('\n', pos);
            if (nl != std::string::npos) {
                size_t end = nl;
                if (end > pos && buf[end - 1] == '\r') --end;
                out.assign(buf, pos, end - pos);
                pos = nl + 1;
                return true;
            }
            if (buf.size() - pos > (1u << 20)) return false;  // a header line this long is an attack or a bug
            if (!fill()) return false;
        }
    }
    bool bytes(size_t n, std::string& out)
    {
        while (buf.size() - pos < n)
            if (!fill()) return false;
        out.assign(buf, pos, n);
        pos += n;
        return true;
    }
};

std::string lower(std::string s)
{
    for (auto& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    return s;
}

std::string upper(std::string s)
{
    for (auto& c : s) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
    return s;
}

const char* reason(int status)
{
    switch (status) {
        case 200: return "OK";
        case 400: return "Bad Request";
        case 404: return "Not Found";
        case 405: return "Method Not Allowed";
        case 409: return "Conflict";
        case 500: return "Internal Server Error";
        case 503: return "Service Unavailable";
        default: return "Status";
    }
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// TcpListener
// ------------------------------------------------------------------------------------------------
int TcpListener::start(const std::string& host, int port, ConnHandler on_conn)
{
    on_conn_ = std::move(on_conn);
    fd_      = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd_ < 0) throw std::runtime_error(std::string("socket() failed: ") + strerror(errno));
    int one = 1;
    setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port   = htons(static_cast<uint16_t>(port));
    if (host.empty() || host == "0.0.0.0" || inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1)
        addr.sin_addr.s_addr = htonl(INADDR_ANY);
    if (::bind(fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd_, 128) != 0) {
        const std::string why = strerror(errno);
        ::close(fd_);
        fd_ = -1;
        throw std::runtime_error("cannot listen on " + host + ":" + std::to_string(port) + ": " + why);
    }
    socklen_t len = sizeof(addr);
    getsockname(fd_, reinterpret_cast<sockaddr*>(&addr), &len);
    port_ = ntohs(addr.sin_port);
    running_.store(true);
    acceptor_ = std::thread([this] { accept_loop(); });
    return port_;
}

void TcpListener::accept_loop()
{
    while (running_.load()) {
        pollfd    p{fd_, POLLIN, 0};
        const int r = ::poll(&p, 1, 200);
        if (r <= 0) continue;
        const int c = ::accept(fd_, nullptr, nullptr);
        if (c < 0) continue;
        int one = 1;
        setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        std::lock_guard<std::mutex> g(mu_);
        if (!running_.load()) {
            ::close(c);
            break;
        }
        conns_.insert(c);
        active_.fetch_add(1);
        std::thread([this, c] {
            on_conn_(c);
            {
                std::lock_guard<std::mutex> g2(mu_);
                if (conns_.erase(c)) ::close(c);
            }
            active_.fetch_sub(1);
        }).detach();
    }
}

void TcpListener::stop()
{
    if (!running_.exchange(false)) return;
    if (acceptor_.joinable()) acceptor_.join();
    {
        std::lock_guard<std::mutex> g(mu_);
        for (int c : conns_) ::shutdown(c, SHUT_RDWR);
    }
    // connection threads are detached; they leave as soon as their socket is shut down
    for (int i = 0; i < 5000 && active_.load() > 0; ++i) usleep(1000);
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
}

// ------------------------------------------------------------------------------------------------
// HttpServer
// ------------------------------------------------------------------------------------------------
int HttpServer::start(const std::string& host, int port, Handler h)
{
    handler_ = std::move(h);
    return listener_.start(host, port, [this](int fd) { serve(fd); });
}

void HttpServer::serve(int fd)
{
    Reader rd{fd};
    while (listener_.running()) {
        std::string line;
        if (!rd.line(line)) return;
        if (line.empty()) continue;
        HttpRequest req;
        {
            const size_t a = line.find(' '), b = line.rfind(' ');
            if (a == std::string::npos || b == a) return;
            req.method = line.substr(0, a);
            req.path   = line.substr(a + 1, b - a - 1);
            const size_t q = req.path.find('?');
            if (q != std::string::npos) req.path.resize(q);
        }
        size_t content_length = 0;
        bool   close_after    = false;
        while (true) {
            if (!rd.line(line)) return;
            if (line.empty()) break;
            const size_t colon = line.find(':');
            if (colon == std::string::npos) continue;
            std::string name = lower(line.substr(0, colon));
            std::string val  = line.substr(colon + 1);
            while (!val.empty() && val.front() == ' ') val.erase(val.begin());
            if (name == "content-length") content_length = static_cast<size_t>(std::strtoull(val.c_str(), nullptr, 10));
            if (name == "connection" && lower(val) == "close") close_after = true;
            req.headers[name] = val;
        }
        if (content_length > (256u << 20)) return;
        if (content_length && !rd.bytes(content_length, req.body)) return;
        HttpResponse rsp;
        try {
            rsp = handler_(req);
        }
        catch (const std::exception& e) {
            rsp.status = 500;
            rsp.body   = std::string("{\"status\":\"error\",\"message\":\"") + e.what() + "\"}";
        }
        std::string out = "HTTP/1.1 " + std::to_string(rsp.status) + " " + reason(rsp.status) + "\r\n";
        out += "Content-Type: " + rsp.content_type + "\r\n";
        out += "Content-Length: " + std::to_string(rsp.body.size()) + "\r\n";
        out += close_after ? "Connection: close\r\n\r\n" : "Connection: keep-alive\r\n\r\n";
        out += rsp.body;
        if (!write_all(fd, out) || close_after) return;
    }
}

// ------------------------------------------------------------------------------------------------
// RespServer
// ------------------------------------------------------------------------------------------------
namespace {

std::string r_simple(const std::string& s) { return "+" + s + "\r\n"; }
std::string r_err(const std::string& s) { return "-" + s + "\r\n"; }
std::string r_int(int64_t v) { return ":" + std::to_string(v) + "\r\n"; }
std::string r_bulk(const std::string& s) { return "$" + std::to_string(s.size()) + "\r\n" + s + "\r\n"; }
std::string r_null() { return "$-1\r\n"; }
std::string r_null_array() { return "*-1\r\n"; }
std::string r_array_hdr(size_t n) { return "*" + std::to_string(n) + "\r\n"; }

std::string r_entries(const std::vector<StreamEntry>& es)
{
    std::string out = r_array_hdr(es.size());
    for (const auto& e : es) {
        out += r_array_hdr(2) + r_bulk(e.id.str()) + r_array_hdr(e.fields.size() * 2);
        for (const auto& f : e.fields) out += r_bulk(f.first) + r_bulk(f.second);
    }
    return out;
}

bool parse_i64(const std::string& s, int64_t& out)
{
    char* end = nullptr;
    errno     = 0;
    long long v = std::strtoll(s.c_str(), &end, 10);
    if (s.empty() || *end != 0 || errno != 0) return false;
    out = v;
    return true;
}

}  // namespace

int RespServer::start(const std::string& host, int port)
{
    return listener_.start(host, port, [this](int fd) { serve(fd); });
}

void RespServer::stop()
{
    store_->interrupt();
    listener_.stop();
}

void RespServer::serve(int fd)
{
    Reader rd{fd};
    while (listener_.running()) {
        std::string line;
        if (!rd.line(line)) return;
        if (line.empty()) continue;
        std::vector<std::string> argv;
        if (line[0] == '*') {
            int64_t n = 0;
            if (!parse_i64(line.substr(1), n) || n < 0 || n > 1 << 20) return;
            for (int64_t i = 0; i < n; ++i) {
                if (!rd.line(line) || line.empty() || line[0] != '$') return;
                int64_t len = 0;
                if (!parse_i64(line.substr(1), len) || len < 0 || len > (512ll << 20)) return;
                std::string arg, crlf;
                if (!rd.bytes(static_cast<size_t>(len), arg) || !rd.bytes(2, crlf)) return;
                argv.push_back(std::move(arg));
            }
        }
        else {
            // inline command
            size_t i = 0;
            while (i < line.size()) {
                while (i < line.size() && line[i] == ' ') ++i;
                size_t j = i;
                while (j < line.size() && line[j] != ' ') ++j;
                if (j > i) argv.push_back(line.substr(i, j - i));
                i = j;
            }
        }
        if (argv.empty()) continue;
        std::string reply;
        try {
            reply = execute(argv);
        }
        catch (const std::exception& e) {
            const std::string m = e.what();
            reply = r_err((m.rfind("ERR", 0) == 0 || m.rfind("WRONGTYPE", 0) == 0) ? m : "ERR " + m);
        }
        if (!write_all(fd, reply)) return;
        if (upper(argv[0]) == "QUIT") return;
    }
}

std::string RespServer::execute(const std::vector<std::string>& argv)
{
    const std::string cmd = upper(argv[0]);
    const size_t      n   = argv.size();
    auto need = [&](size_t k) {
        if (n < k) throw std::runtime_error("ERR wrong number of arguments for '" + argv[0] + "' command");
    };
    KvStore& kv = *store_;

    if (cmd == "PING") return n > 1 ? r_bulk(argv[1]) : r_simple("PONG");
    if (cmd == "ECHO") { need(2); return r_bulk(argv[1]); }
    if (cmd == "QUIT") return r_simple("OK");
    if (cmd == "SELECT" || cmd == "CLIENT" || cmd == "AUTH" || cmd == "HELLO") {
        if (cmd == "HELLO") throw std::runtime_error("ERR unknown command 'HELLO'");  // RESP2 only
        return r_simple("OK");
    }
    if (cmd == "COMMAND") return r_array_hdr(0);
    if (cmd == "INFO") return r_bulk("# Server\r\nredis_version:7.0.0-slime\r\nredis_mode:embedded\r\n");
    if (cmd == "DBSIZE") return r_int(static_cast<int64_t>(kv.size()));
    if (cmd == "FLUSHALL" || cmd == "FLUSHDB") { kv.flush_all(); return r_simple("OK"); }

    if (cmd == "SET") {
        need(3);
        int64_t ttl = -1;
        bool    nx  = false;
        for (size_t i = 3; i < n; ++i) {
            const std::string o = upper(argv[i]);
            if ((o == "EX" || o == "PX") && i + 1 < n) {
                int64_t v = 0;
                if (!parse_i64(argv[++i], v) || v <= 0) throw std::runtime_error("ERR invalid expire time in 'set' command");
                ttl = o == "EX" ? v * 1000 : v;
            }
            else if (o == "NX") nx = true;
            else if (o == "XX" || o == "KEEPTTL") {}
            else throw std::runtime_error("ERR syntax error");
        }
        return kv.set(argv[1], argv[2], ttl, nx) ? r_simple("OK") : r_null();
    }
    if (cmd == "SETEX" || cmd == "PSETEX") {
        need(4);
        int64_t v = 0;
        if (!parse_i64(argv[2], v) || v <= 0) throw std::runtime_error("ERR invalid expire time");
        kv.set(argv[1], argv[3], cmd == "SETEX" ? v * 1000 : v);
        return r_simple("OK");
    }
    if (cmd == "SETNX") { need(3); return r_int(kv.set(argv[1], argv[2], -1, true) ? 1 : 0); }
    if (cmd == "GET") {
        need(2);
        auto v = kv.get(argv[1]);
        return v ? r_bulk(*v) : r_null();
    }
    if (cmd == "MGET") {
        need(2);
        auto vs = kv.mget({argv.begin() + 1, argv.end()});
        std::string out = r_array_hdr(vs.size());
        for (auto& v : vs) out += v ? r_bulk(*v) : r_null();
        return out;
    }
    if (cmd == "DEL" || cmd == "UNLINK") { need(2); return r_int(kv.del({argv.begin() + 1, argv.end()})); }
    if (cmd == "EXISTS") {
        need(2);
        int64_t c = 0;
        for (size_t i = 1; i < n; ++i) c += kv.exists(argv[i]) ? 1 : 0;
        return r_int(c);
    }
    if (cmd == "EXPIRE" || cmd == "PEXPIRE") {
        need(3);
        int64_t v = 0;
        if (!parse_i64(argv[2], v)) throw std::runtime_error("ERR value is not an integer or out of range");
        return r_int(kv.expire(argv[1], cmd == "EXPIRE" ? v * 1000 : v) ? 1 : 0);
    }
    if (cmd == "TTL" || cmd == "PTTL") {
        need(2);
        const int64_t t = kv.pttl(argv[1]);
        return r_int(t < 0 ? t : (cmd == "TTL" ? (t + 999) / 1000 : t));
    }
    if (cmd == "INCR") { need(2); return r_int(kv.incr(argv[1], 1)); }
    if (cmd == "DECR") { need(2); return r_int(kv.incr(argv[1], -1)); }
    if (cmd == "INCRBY") {
        need(3);
        int64_t v = 0;
        if (!parse_i64(argv[2], v)) throw std::runtime_error("ERR value is not an integer or out of range");
        return r_int(kv.incr(argv[1], v));
    }
    if (cmd == "TYPE") { need(2); return r_simple(kv.type_of(argv[1])); }
    if (cmd == "KEYS") {
        need(2);
        auto ks = kv.keys(argv[1]);
        std::string out = r_array_hdr(ks.size());
        for (auto& k : ks) out += r_bulk(k);
        return out;
    }
    if (cmd == "SCAN") {
        need(2);
        int64_t cursor = 0, count = 10;
        if (!parse_i64(argv[1], cursor) || cursor < 0) throw std::runtime_error("ERR invalid cursor");
        std::string pattern = "*";
        for (size_t i = 2; i + 1 < n; i += 2) {
            const std::string o = upper(argv[i]);
            if (o == "MATCH") pattern = argv[i + 1];
            else if (o == "COUNT") {
                if (!parse_i64(argv[i + 1], count) || count <= 0) throw std::runtime_error("ERR syntax error");
            }
        }
        auto res = kv.scan(static_cast<uint64_t>(cursor), pattern, static_cast<size_t>(count));
        std::string out = r_array_hdr(2) + r_bulk(std::to_string(res.first)) + r_array_hdr(res.second.size());
        for (auto& k : res.second) out += r_bulk(k);
        return out;
    }

    // ---- hashes
    if (cmd == "HSET" || cmd == "HMSET") {
        need(4);
        if ((n - 2) % 2 != 0) throw std::runtime_error("ERR wrong number of arguments for 'hset' command");
        std::vector<std::pair<std::string, std::string>> f;
        for (size_t i = 2; i + 1 < n; i += 2) f.emplace_back(argv[i], argv[i + 1]);
        const int64_t added = kv.hset(argv[1], f);
        return cmd == "HMSET" ? r_simple("OK") : r_int(added);
    }
    if (cmd == "HGET") {
        need(3);
        auto v = kv.hget(argv[1], argv[2]);
        return v ? r_bulk(*v) : r_null();
    }
    if (cmd == "HGETALL") {
        need(2);
        auto fs = kv.hgetall(argv[1]);
        std::string out = r_array_hdr(fs.size() * 2);
        for (auto& f : fs) out += r_bulk(f.first) + r_bulk(f.second);
        return out;
    }
    if (cmd == "HDEL") { need(3); return r_int(kv.hdel(argv[1], {argv.begin() + 2, argv.end()})); }

    // ---- lists
    if (cmd == "LPUSH") { need(3); return r_int(kv.lpush(argv[1], {argv.begin() + 2, argv.end()})); }
    if (cmd == "RPUSH") { need(3); return r_int(kv.rpush(argv[1], {argv.begin() + 2, argv.end()})); }
    if (cmd == "LPOP" || cmd == "RPOP") {
        need(2);
        auto v = cmd == "LPOP" ? kv.lpop(argv[1]) : kv.rpop(argv[1]);
        return v ? r_bulk(*v) : r_null();
    }
    if (cmd == "LLEN") { need(2); return r_int(kv.llen(argv[1])); }
    if (cmd == "LRANGE") {
        need(4);
        int64_t a = 0, b = 0;
        if (!parse_i64(argv[2], a) || !parse_i64(argv[3], b)) throw std::runtime_error("ERR value is not an integer or out of range");
        auto vs = kv.lrange(argv[1], a, b);
        std::string out = r_array_hdr(vs.size());
        for (auto& v : vs) out += r_bulk(v);
        return out;
    }
    if (cmd == "BLPOP") {
        need(3);
        const double  secs = std::strtod(argv[n - 1].c_str(), nullptr);
        auto          res  = kv.blpop({argv.begin() + 1, argv.end() - 1}, static_cast<int64_t>(secs * 1000.0));
        if (!res) return r_null_array();
        return r_array_hdr(2) + r_bulk(res->first) + r_bulk(res->second);
    }

    // ---- streams
    if (cmd == "XADD") {
        need(5);
        size_t i = 2, maxlen = 0;
        if (upper(argv[i]) == "MAXLEN") {
            ++i;
            if (i < n && (argv[i] == "~" || argv[i] == "=")) ++i;
            int64_t v = 0;
            if (i >= n || !parse_i64(argv[i], v) || v < 0) throw std::runtime_error("ERR value is not an integer or out of range");
            maxlen = static_cast<size_t>(v);
            ++i;
        }
        if (i >= n) throw std::runtime_error("ERR wrong number of arguments for 'xadd' command");
        const std::string id = argv[i++];
        if ((n - i) == 0 || (n - i) % 2 != 0) throw std::runtime_error("ERR wrong number of arguments for 'xadd' command");
        std::vector<std::pair<std::string, std::string>> f;
        for (; i + 1 < n; i += 2) f.emplace_back(argv[i], argv[i + 1]);
        const std::string got = kv.xadd(argv[1], id, f, maxlen);
        if (got.empty()) throw std::runtime_error("ERR The ID specified in XADD is equal or smaller than the target stream top item");
        return r_bulk(got);
    }
    if (cmd == "XLEN") { need(2); return r_int(kv.xlen(argv[1])); }
    if (cmd == "XRANGE") {
        need(4);
        size_t count = 0;
        if (n >= 6 && upper(argv[4]) == "COUNT") count = static_cast<size_t>(std::strtoull(argv[5].c_str(), nullptr, 10));
        return r_entries(kv.xrange(argv[1], argv[2], argv[3], count));
    }
    if (cmd == "XREAD") {
        size_t  i = 1, count = 0;
        int64_t block = -1;
        while (i < n) {
            const std::string o = upper(argv[i]);
            if (o == "COUNT" && i + 1 < n) { count = static_cast<size_t>(std::strtoull(argv[i + 1].c_str(), nullptr, 10)); i += 2; }
            else if (o == "BLOCK" && i + 1 < n) { if (!parse_i64(argv[i + 1], block) || block < 0) throw std::runtime_error("ERR timeout is not an integer or out of range"); i += 2; }
            else if (o == "STREAMS") { ++i; break; }
            else throw std::runtime_error("ERR syntax error");
        }
        const size_t rest = n - i;
        if (rest == 0 || rest % 2 != 0) throw std::runtime_error("ERR Unbalanced XREAD list of streams: for each stream key an ID or '$' must be specified.");
        std::vector<std::pair<std::string, std::string>> ki;
        for (size_t k = 0; k < rest / 2; ++k) ki.emplace_back(argv[i + k], argv[i + rest / 2 + k]);
        auto res = kv.xread(ki, count, block);
        if (res.empty()) return r_null_array();
        std::string out = r_array_hdr(res.size());
        for (auto& s : res) out += r_array_hdr(2) + r_bulk(s.first) + r_entries(s.second);
        return out;
    }

    if (cmd == "PUBLISH") { need(3); return r_int(kv.publish(argv[1], argv[2])); }

    throw std::runtime_error("ERR unknown command '" + argv[0] + "'");
}

}  // namespace ctrl
}  // namespace slime
