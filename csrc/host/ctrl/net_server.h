// Two small socket servers for the control plane, both thread-per-connection:
//   HttpServer  HTTP/1.1 with keep-alive, Content-Length bodies, a handler per request
//   RespServer  the RESP2 protocol subset that maps onto KvStore, so that any Redis client
//               (or the bundled Python client) can use the embedded store
// Neither depends on a third-party library.
#pragma once

#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "ctrl/kvstore.h"

namespace slime {
namespace ctrl {

// Listening socket plus accept loop shared by both servers.
class TcpListener {
public:
    using ConnHandler = std::function<void(int fd)>;
    ~TcpListener() { stop(); }
    // port 0 picks a free port. Returns the bound port; throws on failure.
    int  start(const std::string& host, int port, ConnHandler on_conn);
    void stop();
    int  port() const { return port_; }
    bool running() const { return running_.load(); }

private:
    void accept_loop();
    int  fd_   = -1;
    int  port_ = 0;
    std::atomic<bool> running_{false};
    ConnHandler       on_conn_;
    std::thread       acceptor_;
    std::mutex        mu_;
    std::set<int>     conns_;
    std::atomic<int>  active_{0};
};

struct HttpRequest {
    std::string method, path, body;
    std::map<std::string, std::string> headers;  // lower-case names
};

struct HttpResponse {
    int         status = 200;
    std::string content_type = "application/json";
    std::string body;
};

class HttpServer {
public:
    using Handler = std::function<HttpResponse(const HttpRequest&)>;
    int  start(const std::string& host, int port, Handler h);
    void stop() { listener_.stop(); }
    int  port() const { return listener_.port(); }

private:
    void serve(int fd);
    Handler     handler_;
    TcpListener listener_;
};

class RespServer {
public:
    explicit RespServer(std::shared_ptr<KvStore> store): store_(std::move(store)) {}
    int  start(const std::string& host, int port);
    void stop();
    int  port() const { return listener_.port(); }
    // Executes one command (argv[0] is the command name) and returns the RESP-encoded reply.
    std::string execute(const std::vector<std::string>& argv);

private:
    void serve(int fd);
    std::shared_ptr<KvStore> store_;
    TcpListener              listener_;
};

}  // namespace ctrl
}  // namespace slime
