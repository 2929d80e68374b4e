#include "ctrl/nanoctrl.h"

#include <chrono>
#include <cstdio>
#include <set>

#include "core/log.h"

namespace slime {
namespace ctrl {

namespace {

int64_t unix_secs()
{
    return std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

HttpResponse json_response(const Json& j, int status = 200)
{
    HttpResponse r;
    r.status = status;
    r.body   = j.dump();
    return r;
}

Json ok(const std::string& message = "")
{
    Json j      = Json::object();
    j["status"] = "ok";
    if (!message.empty()) j["message"] = message;
    return j;
}

std::string require_string(const Json& body, const char* field)
{
    if (!body[field].is_string() || body[field].as_string().empty())
        throw HttpError(400, std::string("missing field '") + field + "'");
    return body[field].as_string();
}

}  // namespace

NanoCtrl::NanoCtrl(): store_(std::make_shared<KvStore>()) {}

NanoCtrl::~NanoCtrl()
{
    stop();
}

void NanoCtrl::start(const std::string& host, int http_port, int resp_port, const std::string& public_host)
{
    if (running_) return;
    bind_host_   = host;
    public_host_ = public_host;
    resp_        = std::make_unique<RespServer>(store_);
    resp_->start(host, resp_port);
    http_.start(host, http_port, [this](const HttpRequest& r) { return handle(r); });
    running_ = true;
    SLIME_LOG_INFO("nanoctrl listening: http ", host, ":", http_.port(), " store ", host, ":", resp_->port());
}

void NanoCtrl::stop()
{
    if (!running_) return;
    running_ = false;
    http_.stop();
    if (resp_) resp_->stop();
}

std::string NanoCtrl::redis_host_for(const HttpRequest& req) const
{
    // What a remote client should dial: an explicit public host wins; a wildcard or loopback bind is
    // replaced by the host name the client used to reach us (its Host header).
    if (!public_host_.empty()) return public_host_;
    if (const char* env = std::getenv("REDIS_PUBLIC_ADDRESS"); env && *env) return env;
    const bool local_bind = bind_host_.empty() || bind_host_ == "0.0.0.0" || bind_host_ == "127.0.0.1" || bind_host_ == "localhost";
    if (local_bind) {
        auto it = req.headers.find("host");
        if (it != req.headers.end() && !it->second.empty()) {
            std::string h = it->second;
            const size_t colon = h.rfind(':');
            if (colon != std::string::npos) h.resize(colon);
            if (!h.empty()) return h;
        }
        return "127.0.0.1";
    }
    return bind_host_;
}

// ------------------------------------------------------------------------------------------------
// operations
// ------------------------------------------------------------------------------------------------
std::string NanoCtrl::register_agent(const std::string& scope, const Json& body)
{
    std::lock_guard<std::mutex> g(script_mu_);
    std::string name;
    const bool  alias_given = body["alias"].is_string() && !body["alias"].as_string().empty();
    if (alias_given) {
        name = body["alias"].as_string();
    }
    else {
        const int64_t c = store_->incr(scoped_key(scope, "agent_name_counter"));
        char          hex[32];
        snprintf(hex, sizeof(hex), "%llx", static_cast<long long>(c));
        name = body["name_prefix"].string_or("agent") + "-" + hex;
    }
    const std::string key = scoped_key(scope, "agent:" + name);
    if (alias_given && store_->exists(key)) throw HttpError(409, "Peer agent alias '" + name + "' already exists in this scope");
    std::vector<std::pair<std::string, std::string>> f;
    f.emplace_back("addr", body["address"].string_or(""));
    f.emplace_back("updated_at", std::to_string(unix_secs()));
    f.emplace_back("memory_keys", "[]");
    if (body["device"].is_string()) f.emplace_back("device", body["device"].as_string());
    if (body["ib_port"].is_number()) f.emplace_back("ib_port", std::to_string(body["ib_port"].as_int()));
    if (body["link_type"].is_string()) f.emplace_back("link_type", body["link_type"].as_string());
    if (!body["resource"].is_null()) {
        const std::string r = body["resource"].dump();
        f.emplace_back("resource", r);
        f.emplace_back("topology", r);
    }
    store_->hset(key, f);
    store_->expire(key, kEntityTtlSecs * 1000ll);
    return name;
}

Json NanoCtrl::list_agents(const std::string& scope)
{
    Json              out    = Json::array();
    const std::string prefix = scoped_key(scope, "agent:");
    for (const auto& key : store_->keys(prefix + "*")) {
        std::map<std::string, std::string> h;
        for (auto& kv : store_->hgetall(key)) h[kv.first] = kv.second;
        if (!h.count("addr")) continue;
        Json a         = Json::object();
        a["name"]      = key.substr(prefix.size());
        a["device"]    = h.count("device") ? h["device"] : "";
        a["ib_port"]   = h.count("ib_port") ? Json(h["ib_port"]).as_int(1) : 1;
        a["link_type"] = h.count("link_type") ? h["link_type"] : "";
        a["address"]   = h["addr"];
        Json res, mk;
        a["resource"]    = (h.count("resource") && Json::try_parse(h["resource"], res)) ? res : Json();
        a["memory_keys"] = (h.count("memory_keys") && Json::try_parse(h["memory_keys"], mk) && mk.is_array()) ? mk : Json::array();
        out.push_back(a);
    }
    return out;
}

void NanoCtrl::cleanup_agent(const std::string& scope, const std::string& agent)
{
    std::lock_guard<std::mutex> g(script_mu_);
    std::set<std::string> notify;
    const std::string     spec_key = scoped_key(scope, "spec:topology:" + agent);
    auto targets_of = [](const std::string& text) {
        std::vector<std::string> out;
        Json spec;
        if (Json::try_parse(text, spec))
            for (const auto& p : spec["target_peers"].items())
                if (p.is_string()) out.push_back(p.as_string());
        return out;
    };
    if (auto own = store_->get(spec_key))
        for (auto& p : targets_of(*own)) notify.insert(p);
    const std::string spec_prefix = scoped_key(scope, "spec:topology:");
    for (const auto& key : store_->keys(spec_prefix + "*")) {
        if (key == spec_key) continue;
        auto text = store_->get(key);
        if (!text) continue;
        for (auto& p : targets_of(*text))
            if (p == agent) notify.insert(key.substr(spec_prefix.size()));
    }
    std::vector<std::string> doomed{scoped_key(scope, "agent:" + agent), spec_key, scoped_key(scope, "inbox:" + agent)};
    for (const std::string& pattern : {"exchange:" + agent + ":*", "exchange:*:" + agent, "mr:" + agent + ":*"})
        for (auto& k : store_->keys(scoped_key(scope, pattern))) doomed.push_back(k);
    store_->del(doomed);
    Json ev    = Json::object();
    ev["type"] = "cleanup";
    ev["peer"] = agent;
    for (const auto& peer : notify) {
        if (peer == agent) continue;
        store_->lpush(scoped_key(scope, "inbox:" + peer), {ev.dump()});
    }
}

void NanoCtrl::save_topology(const std::string& scope, const std::string& agent, const Json& spec)
{
    std::lock_guard<std::mutex> g(script_mu_);
    auto announce = [&](const std::string& to, const std::string& peer) {
        store_->xadd(scoped_key(scope, "stream:" + to), "*",
                     {{"type", "connect_peer"}, {"peer", peer}, {"timestamp", std::to_string(unix_secs())}}, 1000);
    };
    Json stored            = Json::object();
    stored["target_peers"] = spec["target_peers"].is_array() ? spec["target_peers"] : Json::array();
    if (!spec["min_bw"].is_null()) stored["min_bw"] = spec["min_bw"];
    stored["symmetric"] = spec["symmetric"].as_bool(false);
    store_->set(scoped_key(scope, "spec:topology:" + agent), stored.dump());
    for (const auto& p : stored["target_peers"].items()) {
        if (!p.is_string()) continue;
        announce(agent, p.as_string());
        if (stored["symmetric"].as_bool()) {
            // the peer's own spec gains this agent, and it is told to connect back
            const std::string pk = scoped_key(scope, "spec:topology:" + p.as_string());
            Json              ps = Json::object();
            if (auto cur = store_->get(pk)) Json::try_parse(*cur, ps);
            if (!ps["target_peers"].is_array()) ps["target_peers"] = Json::array();
            bool present = false;
            for (const auto& q : ps["target_peers"].items()) present = present || (q.is_string() && q.as_string() == agent);
            if (!present) ps["target_peers"].push_back(agent);
            store_->set(pk, ps.dump());
            announce(p.as_string(), agent);
        }
    }
}

int64_t NanoCtrl::register_entity(const std::string& scope, const Json& body)
{
    std::lock_guard<std::mutex> g(script_mu_);
    const std::string type = body["entity_type"].string_or("service");
    const std::string id   = require_string(body, "entity_id");
    const std::string kind = body["kind"].string_or("");
    Json info              = Json::object();
    info["entity_type"]    = type;
    info["entity_id"]      = id;
    info["id"]             = id;
    info["kind"]           = kind;
    info["endpoint"]       = body["endpoint"];
    info["metadata"]       = body["metadata"].is_null() ? Json::object() : body["metadata"];
    info["resource"]       = body["resource"];
    const std::string key  = scoped_key(scope, type + ":" + id);
    store_->del({key});
    store_->hset(key, {{"entity_type", type},
                       {"entity_id", id},
                       {"kind", kind},
                       {"endpoint", body["endpoint"].is_null() ? "" : body["endpoint"].dump()},
                       {"metadata", info["metadata"].dump()},
                       {"resource", body["resource"].is_null() ? "" : body["resource"].dump()},
                       {"info", info.dump()}});
    store_->expire(key, kEntityTtlSecs * 1000ll);
    const int64_t rev = store_->incr(scoped_key(scope, "nano_meta:" + type + "_revision"));
    Json ev           = Json::object();
    ev["event_type"]  = "ADD";
    ev["entity_type"] = type;
    ev["entity_id"]   = id;
    ev["kind"]        = kind;
    ev["timestamp"]   = static_cast<long long>(unix_secs());
    ev["revision"]    = static_cast<long long>(rev);
    ev["payload"]     = info;
    store_->publish(scoped_key(scope, "nano_events:" + type + "_update"), ev.dump());
    return rev;
}

int64_t NanoCtrl::unregister_entity(const std::string& scope, const std::string& type, const std::string& id)
{
    std::lock_guard<std::mutex> g(script_mu_);
    const std::string key = scoped_key(scope, type + ":" + id);
    if (!store_->exists(key)) return 0;
    store_->del({key});
    const int64_t rev = store_->incr(scoped_key(scope, "nano_meta:" + type + "_revision"));
    Json ev           = Json::object();
    ev["event_type"]  = "REMOVE";
    ev["entity_type"] = type;
    ev["entity_id"]   = id;
    ev["timestamp"]   = static_cast<long long>(unix_secs());
    ev["revision"]    = static_cast<long long>(rev);
    store_->publish(scoped_key(scope, "nano_events:" + type + "_update"), ev.dump());
    return rev;
}

bool NanoCtrl::heartbeat(const std::string& scope, const std::string& type, const std::string& id)
{
    return store_->expire(scoped_key(scope, type + ":" + id), kEntityTtlSecs * 1000ll);
}

// ------------------------------------------------------------------------------------------------
// routing
// ------------------------------------------------------------------------------------------------
HttpResponse NanoCtrl::handle(const HttpRequest& req)
{
    try {
        if (req.path == "/" && req.method == "GET") {
            HttpResponse r;
            r.content_type = "text/plain";
            r.body         = "NanoCtrl Server Running";
            return r;
        }
        if (req.method != "POST") throw HttpError(req.path == "/" ? 405 : 404, "no such route");
        Json body = Json::object();
        if (!req.body.empty() && !Json::try_parse(req.body, body)) throw HttpError(400, "request body is not valid JSON");
        if (!body.is_object()) throw HttpError(400, "request body must be a JSON object");
        const std::string scope = body["scope"].string_or("");

        if (req.path == "/heartbeat") {
            const std::string type = require_string(body, "entity_type"), id = require_string(body, "entity_id");
            Json j = Json::object();
            if (heartbeat(scope, type, id)) {
                j["status"]  = "ok";
                j["message"] = "heartbeat accepted";
            }
            else {
                j["status"]  = "not_found";
                j["message"] = type + " '" + id + "' is not registered";
            }
            return json_response(j);
        }
        if (req.path == "/start_peer_agent") {
            if (!body["address"].is_string()) throw HttpError(400, "missing field 'address'");
            const std::string name = register_agent(scope, body);
            Json j                 = Json::object();
            j["status"]            = "ok";
            j["name"]              = name;
            j["redis_address"]     = redis_host_for(req) + ":" + std::to_string(resp_port());
            if (!body["resource"].is_null()) j["resource"] = body["resource"];
            return json_response(j);
        }
        if (req.path == "/query") return json_response(list_agents(scope));
        if (req.path == "/cleanup") {
            const std::string agent = require_string(body, "agent_name");
            cleanup_agent(scope, agent);
            return json_response(ok("Cleaned up agent " + agent));
        }
        if (req.path.rfind("/v1/desired_topology/", 0) == 0) {
            const std::string agent = req.path.substr(strlen("/v1/desired_topology/"));
            if (agent.empty()) throw HttpError(400, "missing agent id");
            if (!body["target_peers"].is_array()) throw HttpError(400, "missing field 'target_peers'");
            save_topology(scope, agent, body);
            return json_response(ok());
        }
        if (req.path == "/register_mr") {
            const std::string agent = require_string(body, "agent_name"), mr = require_string(body, "mr_name");
            Json v      = Json::object();
            v["addr"]   = body["addr"];
            v["length"] = body["length"];
            v["rkey"]   = body["rkey"];
            v["lkey"]   = body["lkey"].is_null() ? Json(0) : body["lkey"];
            store_->set(scoped_key(scope, "mr:" + agent + ":" + mr), v.dump());
            return json_response(ok());
        }
        if (req.path == "/get_mr_info") {
            const std::string dst = require_string(body, "dst"), mr = require_string(body, "mr_name");
            Json j = Json::object(), v;
            auto text    = store_->get(scoped_key(scope, "mr:" + dst + ":" + mr));
            j["mr_info"] = (text && Json::try_parse(*text, v)) ? v : Json();
            return json_response(j);
        }
        if (req.path == "/register") {
            const int64_t rev = register_entity(scope, body);
            return json_response(ok("registered (revision " + std::to_string(rev) + ")"));
        }
        if (req.path == "/unregister") {
            const std::string type = body["entity_type"].string_or("service"), id = require_string(body, "entity_id");
            const int64_t rev = unregister_entity(scope, type, id);
            return json_response(ok(rev == 0 ? "not registered; nothing to do" : "unregistered"));
        }
        if (req.path == "/get_entity_info") {
            const std::string type = body["entity_type"].string_or("service"), id = require_string(body, "entity_id");
            Json j = Json::object(), v;
            auto text = store_->hget(scoped_key(scope, type + ":" + id), "info");
            if (text && Json::try_parse(*text, v)) {
                j["status"]      = "ok";
                j["entity_info"] = v;
            }
            else {
                j["status"]      = "not_found";
                j["entity_info"] = Json();
            }
            return json_response(j);
        }
        if (req.path == "/list_entities") {
            const std::string type = body["entity_type"].string_or(""), kind = body["kind"].string_or("");
            Json list = Json::array();
            for (const auto& key : store_->keys(scoped_key(scope, type.empty() ? "*:*" : type + ":*"))) {
                if (store_->type_of(key) != "hash") continue;
                auto text = store_->hget(key, "info");
                Json v;
                if (!text || !Json::try_parse(*text, v)) continue;
                if (!kind.empty() && v["kind"].string_or("") != kind) continue;
                list.push_back(v);
            }
            Json j        = ok();
            j["entities"] = list;
            return json_response(j);
        }
        if (req.path == "/get_redis_address") {
            Json j             = ok();
            j["redis_address"] = "redis://" + redis_host_for(req) + ":" + std::to_string(resp_port());
            return json_response(j);
        }
        throw HttpError(404, "no such route: " + req.path);
    }
    catch (const HttpError& e) {
        Json j       = Json::object();
        j["status"]  = "error";
        j["message"] = e.what();
        return json_response(j, e.status);
    }
    catch (const std::exception& e) {
        Json j       = Json::object();
        j["status"]  = "error";
        j["message"] = e.what();
        return json_response(j, 500);
    }
}

}  // namespace ctrl
}  // namespace slime
