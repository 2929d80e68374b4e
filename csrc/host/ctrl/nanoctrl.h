// NanoCtrl: the registration / discovery control plane. Same HTTP routes, JSON bodies,
// status codes and key schema as the reference's Rust server (NanoCtrl/src/main.rs:169-194,
// NanoCtrl/src/redis_repo.rs, NanoCtrl/lua/*.lua in the reference), implemented in C++ on
// an embedded KvStore that is also served over RESP2, so one process provides what the
// reference splits between NanoCtrl and an external Redis. It can run inside a Python
// process (tests, single-node jobs) or as the stand-alone `nanoctrl` binary.
//
// Routes: GET /, POST /heartbeat, /start_peer_agent, /query, /cleanup,
// /v1/desired_topology/{agent}, /register_mr, /get_mr_info, /register, /unregister,
// /get_entity_info, /list_entities, /get_redis_address. Every body may carry "scope";
// a non-empty scope prefixes every key with "{scope}:".
#pragma once

#include <memory>
#include <mutex>
#include <string>

#include "core/json.hpp"
#include "ctrl/kvstore.h"
#include "ctrl/net_server.h"

namespace slime {
namespace ctrl {

constexpr int kEntityTtlSecs = 60;

class NanoCtrl {
public:
    NanoCtrl();
    ~NanoCtrl();

    // Starts the HTTP and RESP listeners (port 0 = pick a free one). public_host is what
    // clients are told to use for the store; empty = derive it from the request / bind host.
    void start(const std::string& host = "127.0.0.1", int http_port = 0, int resp_port = 0, const std::string& public_host = "");
    void stop();
    bool running() const { return running_; }
    int  http_port() const { return http_.port(); }
    int  resp_port() const { return resp_ ? resp_->port() : 0; }
    const std::shared_ptr<KvStore>& store() const { return store_; }

    // The route dispatcher, callable without sockets (unit tests drive it directly).
    HttpResponse handle(const HttpRequest& req);

    // Operations behind the routes.
    std::string register_agent(const std::string& scope, const Json& body);  // returns the name; throws Conflict
    Json        list_agents(const std::string& scope);
    void        cleanup_agent(const std::string& scope, const std::string& agent);
    void        save_topology(const std::string& scope, const std::string& agent, const Json& spec);
    int64_t     register_entity(const std::string& scope, const Json& body);
    int64_t     unregister_entity(const std::string& scope, const std::string& type, const std::string& id);
    bool        heartbeat(const std::string& scope, const std::string& type, const std::string& id);

    static std::string scoped_key(const std::string& scope, const std::string& suffix)
    {
        return scope.empty() ? suffix : scope + ":" + suffix;
    }

private:
    std::string redis_host_for(const HttpRequest& req) const;

    std::shared_ptr<KvStore>    store_;
    HttpServer                  http_;
    std::unique_ptr<RespServer> resp_;
    std::mutex                  script_mu_;  // makes each multi-command operation atomic, like a server-side script
    std::string                 bind_host_, public_host_;
    bool                        running_ = false;
};

struct HttpError: public std::runtime_error {
    int status;
    HttpError(int s, const std::string& m): std::runtime_error(m), status(s) {}
};

}  // namespace ctrl
}  // namespace slime
