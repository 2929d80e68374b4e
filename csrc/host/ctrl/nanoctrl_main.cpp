// The stand-alone `nanoctrl` program:
//   nanoctrl server [--host H] [--port P] [--redis-port R] [--public-host X]   run in the foreground
//   nanoctrl start  [same flags]      detach a server; pid / meta / log files under the runtime directory
//   nanoctrl status                   is the detached server alive and healthy?
//   nanoctrl stop [--force]           terminate it (SIGTERM, or SIGKILL with --force)
//   nanoctrl obs {status|peers|nics|links} [--redis-url U] [--scope S] [--stale-ms 45000] [--json]
// Same commands and runtime-directory rules as the reference's Rust binary
// (NanoCtrl/src/main.rs:45-57,242-429 and NanoCtrl/src/obs.rs:92-266 in the reference): the directory is
// $NANOCTRL_RUNTIME_DIR, else $XDG_RUNTIME_DIR/nanoctrl, else /tmp/nanoctrl. The store that the
// reference expects at --redis-url is built in and listens on --redis-port.
#include <arpa/inet.h>
#include <chrono>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <fstream>
#include <iostream>
#include <netdb.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <sys/wait.h>
#include <thread>
#include <unistd.h>

#include "ctrl/nanoctrl.h"
#include "ctrl/obs_view.h"

using namespace slime;
using namespace slime::ctrl;

namespace {

volatile std::sig_atomic_t g_stop = 0;
void on_signal(int) { g_stop = 1; }

std::string runtime_dir()
{
    if (const char* d = std::getenv("NANOCTRL_RUNTIME_DIR"); d && *d) return d;
    if (const char* x = std::getenv("XDG_RUNTIME_DIR"); x && *x) return std::string(x) + "/nanoctrl";
    return "/tmp/nanoctrl";
}

struct Flags {
    std::string host = "0.0.0.0", public_host, redis_url, scope;
    int         port = 3000, redis_port = 6379, stale_ms = 45000;
    bool        force = false, json = false;
    std::vector<std::string> positional;
};

Flags parse(int argc, char** argv, int first)
{
    Flags f;
    if (const char* u = std::getenv("NANOCTRL_REDIS_URL"); u && *u) f.redis_url = u;
    if (const char* s = std::getenv("NANOCTRL_SCOPE"); s && *s) f.scope = s;
    for (int i = first; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&]() -> std::string {
            if (i + 1 >= argc) {
                fprintf(stderr, "nanoctrl: %s needs a value\n", a.c_str());
                exit(2);
            }
            return argv[++i];
        };
        if (a == "--host") f.host = next();
        else if (a == "--port") f.port = std::atoi(next().c_str());
        else if (a == "--redis-port") f.redis_port = std::atoi(next().c_str());
        else if (a == "--public-host") f.public_host = next();
        else if (a == "--redis-url") f.redis_url = next();
        else if (a == "--scope") f.scope = next();
        else if (a == "--stale-ms") f.stale_ms = std::atoi(next().c_str());
        else if (a == "--force") f.force = true;
        else if (a == "--json") f.json = true;
        else f.positional.push_back(a);
    }
    return f;
}

bool http_healthy(const std::string& host, int port)
{
    addrinfo hints{}, *res = nullptr;
    hints.ai_family   = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    const std::string h = (host == "0.0.0.0" || host.empty()) ? "127.0.0.1" : host;
    if (getaddrinfo(h.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res) return false;
    int  fd = ::socket(AF_INET, SOCK_STREAM, 0);
    bool ok = false;
    if (fd >= 0 && ::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
        const char* req = "GET / HTTP/1.1\r\nHost: x\r\nConnection: close\r\n\r\n";
        if (::send(fd, req, strlen(req), MSG_NOSIGNAL) > 0) {
            char    buf[512];
            ssize_t n = ::recv(fd, buf, sizeof(buf) - 1, 0);
            if (n > 0) {
                buf[n] = 0;
                ok     = strstr(buf, " 200 ") != nullptr;
            }
        }
    }
    if (fd >= 0) ::close(fd);
    freeaddrinfo(res);
    return ok;
}

int run_server(const Flags& f)
{
    std::signal(SIGINT, on_signal);
    std::signal(SIGTERM, on_signal);
    NanoCtrl srv;
    try {
        srv.start(f.host, f.port, f.redis_port, f.public_host);
    }
    catch (const std::exception& e) {
        fprintf(stderr, "nanoctrl: %s\n", e.what());
        return 1;
    }
    printf("NanoCtrl listening on http://%s:%d (store on port %d)\n", f.host.c_str(), srv.http_port(), srv.resp_port());
    fflush(stdout);
    while (!g_stop) std::this_thread::sleep_for(std::chrono::milliseconds(100));
    srv.stop();
    return 0;
}

bool read_meta(Json& meta)
{
    std::ifstream in(runtime_dir() + "/nanoctrl.json");
    if (!in) return false;
    std::string text((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    return Json::try_parse(text, meta);
}

int cmd_start(const Flags& f, const char* self)
{
    const std::string dir = runtime_dir();
    ::mkdir(dir.c_str(), 0755);
    Json meta;
    if (read_meta(meta) && ::kill(static_cast<pid_t>(meta["pid"].as_int()), 0) == 0) {
        printf("nanoctrl is already running (pid %lld)\n", static_cast<long long>(meta["pid"].as_int()));
        return 0;
    }
    const std::string log = dir + "/nanoctrl.log";
    pid_t pid = ::fork();
    if (pid < 0) {
        perror("fork");
        return 1;
    }
    if (pid == 0) {
        ::setsid();
        int fd = ::open(log.c_str(), O_WRONLY | O_CREAT | O_APPEND, 0644);
        if (fd >= 0) {
            ::dup2(fd, 1);
            ::dup2(fd, 2);
        }
        int devnull = ::open("/dev/null", O_RDONLY);
        if (devnull >= 0) ::dup2(devnull, 0);
        std::vector<std::string> args = {self, "server", "--host", f.host, "--port", std::to_string(f.port), "--redis-port",
                                         std::to_string(f.redis_port)};
        if (!f.public_host.empty()) {
            args.push_back("--public-host");
            args.push_back(f.public_host);
        }
        std::vector<char*> cargs;
        for (auto& a : args) cargs.push_back(const_cast<char*>(a.c_str()));
        cargs.push_back(nullptr);
        ::execv(self, cargs.data());
        _exit(127);
    }
    Json m        = Json::object();
    m["pid"]      = static_cast<long long>(pid);
    m["host"]     = f.host;
    m["port"]     = f.port;
    m["redis_port"] = f.redis_port;
    m["log"]      = log;
    std::ofstream(dir + "/nanoctrl.json") << m.dump(2) << "\n";
    std::ofstream(dir + "/nanoctrl.pid") << pid << "\n";
    for (int i = 0; i < 50; ++i) {
        if (http_healthy(f.host, f.port)) {
            printf("nanoctrl started (pid %d), http://%s:%d, log %s\n", pid, f.host.c_str(), f.port, log.c_str());
            return 0;
        }
        int status = 0;
        if (::waitpid(pid, &status, WNOHANG) == pid) break;
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    fprintf(stderr, "nanoctrl did not become healthy; see %s\n", log.c_str());
    return 1;
}

int cmd_status()
{
    Json meta;
    if (!read_meta(meta)) {
        printf("nanoctrl: not running (no metadata in %s)\n", runtime_dir().c_str());
        return 1;
    }
    const pid_t pid   = static_cast<pid_t>(meta["pid"].as_int());
    const bool  alive = ::kill(pid, 0) == 0;
    const bool  ok    = alive && http_healthy(meta["host"].string_or("127.0.0.1"), static_cast<int>(meta["port"].as_int()));
    printf("nanoctrl: pid %d %s, http://%s:%lld %s\n", pid, alive ? "alive" : "dead", meta["host"].string_or("?").c_str(),
           static_cast<long long>(meta["port"].as_int()), ok ? "healthy" : "unreachable");
    return ok ? 0 : 1;
}

int cmd_stop(bool force)
{
    Json meta;
    if (!read_meta(meta)) {
        printf("nanoctrl: not running\n");
        return 0;
    }
    const pid_t pid = static_cast<pid_t>(meta["pid"].as_int());
    if (::kill(pid, force ? SIGKILL : SIGTERM) != 0) {
        printf("nanoctrl: pid %d is already gone\n", pid);
    }
    else {
        for (int i = 0; i < 50 && ::kill(pid, 0) == 0; ++i) {
            ::waitpid(pid, nullptr, WNOHANG);
            std::this_thread::sleep_for(std::chrono::milliseconds(100));
        }
        printf("nanoctrl: stopped pid %d\n", pid);
    }
    const std::string dir = runtime_dir();
    ::unlink((dir + "/nanoctrl.json").c_str());
    ::unlink((dir + "/nanoctrl.pid").c_str());
    return 0;
}

void usage()
{
    fputs("usage: nanoctrl {server|start|status|stop|obs} [options]\n"
          "  server|start: --host H --port P --redis-port R [--public-host X]\n"
          "  stop: [--force]\n"
          "  obs {status|peers|nics|links}: [--redis-url host:port] [--scope S] [--stale-ms N] [--json]\n",
          stderr);
}

}  // namespace

int main(int argc, char** argv)
{
    if (argc < 2) {
        usage();
        return 2;
    }
    const std::string cmd = argv[1];
    const Flags       f   = parse(argc, argv, 2);
    if (cmd == "server") return run_server(f);
    if (cmd == "start") {
        char self[4096];
        ssize_t n = ::readlink("/proc/self/exe", self, sizeof(self) - 1);
        if (n <= 0) {
            fprintf(stderr, "nanoctrl: cannot locate own executable\n");
            return 1;
        }
        self[n] = 0;
        return cmd_start(f, self);
    }
    if (cmd == "status") return cmd_status();
    if (cmd == "stop") return cmd_stop(f.force);
    if (cmd == "obs") {
        std::string address = f.redis_url;
        if (address.empty()) {
            Json meta;
            address = read_meta(meta) ? "127.0.0.1:" + std::to_string(meta["redis_port"].as_int()) : "127.0.0.1:6379";
        }
        const std::string view = f.positional.empty() ? "status" : f.positional[0];
        return obs_view_main(address, f.scope, view, f.stale_ms, f.json);
    }
    usage();
    return 2;
}
