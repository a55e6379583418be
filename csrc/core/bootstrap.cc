#include "bootstrap.h"
#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <algorithm>
#include <fcntl.h>
#include <fstream>
#include <ifaddrs.h>
#include <net/if.h>
#include <set>
#include <sstream>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <random>
#include <sys/socket.h>
#include <sys/un.h>
#include <thread>
#include <unistd.h>
#include "config.h"
#include "json.h"
#include "log.h"

namespace hccl {
namespace {

constexpr uint32_t kHelloMagic = 0x68656c6fu;
struct Hello { uint32_t magic; uint32_t rank; uint32_t nRanks; uint32_t pad; uint64_t uniqueId; };
struct ReqHeader { uint32_t magic; uint32_t seq; uint64_t bytes; };

bool WriteAll(int fd, const void* buf, size_t n)
{
    const char* p = (const char*)buf;
    while (n > 0) {
        ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w < 0) { if (errno == EINTR) continue; return false; }
        p += w; n -= (size_t)w;
    }
    return true;
}
// timeoutMs < 0: wait forever
bool ReadAll(int fd, void* buf, size_t n, int timeoutMs)
{
    char* p = (char*)buf;
    while (n > 0) {
        struct pollfd pf = {fd, POLLIN, 0};
        int pr = ::poll(&pf, 1, timeoutMs);
        if (pr == 0) return false;
        if (pr < 0) { if (errno == EINTR) continue; return false; }
        ssize_t r = ::recv(fd, p, n, 0);
        if (r == 0) return false;
        if (r < 0) { if (errno == EINTR || errno == EAGAIN) continue; return false; }
        p += r; n -= (size_t)r;
    }
    return true;
}

// Relay: accepts nRanks connections, then for every round gathers one request of
// equal size from each rank and answers with the concatenation.
void RelayThread(int listenFd, uint64_t uniqueId, std::shared_ptr<std::set<uint32_t>> allowed)
{
    std::vector<int> fds;
    uint32_t nRanks = 0;
    std::vector<int> byRank;
    // accept phase: the first hello tells how many ranks to expect
    for (;;) {
        struct pollfd pf = {listenFd, POLLIN, 0};
        int pr = ::poll(&pf, 1, 7200 * 1000);
        if (pr <= 0) { if (pr < 0 && errno == EINTR) continue; break; }
        struct sockaddr_in from;
        socklen_t fromLen = sizeof(from);
        int fd = ::accept(listenFd, (struct sockaddr*)&from, &fromLen);
        if (fd < 0) continue;
        if (allowed && !allowed->count(from.sin_addr.s_addr)) {
            // trust list (HCCL_WHITELIST_DISABLE=0): an address that is not listed never gets as far as the hello
            char text[INET_ADDRSTRLEN] = {0};
            inet_ntop(AF_INET, &from.sin_addr, text, sizeof(text));
            HCCL_WARNING("rendezvous: connection from %s refused, the address is not in HCCL_WHITELIST_FILE", text);
            ::close(fd);
            continue;
        }
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        Hello h;
        if (!ReadAll(fd, &h, sizeof(h), 10000) || h.magic != kHelloMagic || h.uniqueId != uniqueId || h.nRanks == 0 ||
            h.rank >= h.nRanks || (nRanks != 0 && h.nRanks != nRanks)) {
            ::close(fd);
            continue;
        }
        if (nRanks == 0) { nRanks = h.nRanks; byRank.assign(nRanks, -1); }
        if (byRank[h.rank] != -1) { ::close(fd); continue; }
        byRank[h.rank] = fd;
        bool all = true;
        for (int f : byRank) all = all && f != -1;
        if (all) break;
    }
    ::close(listenFd);
    if (nRanks == 0) return;
    for (int f : byRank) if (f == -1) { for (int g : byRank) if (g != -1) ::close(g); return; }
    // tell everyone the group is complete
    for (int f : byRank) { uint32_t ok = 1; WriteAll(f, &ok, sizeof(ok)); }
    std::vector<char> gathered;
    for (;;) {
        bool fail = false;
        uint64_t bytes = 0;
        uint32_t seq = 0;
        for (uint32_t r = 0; r < nRanks && !fail; ++r) {
            ReqHeader h;
            if (!ReadAll(byRank[r], &h, sizeof(h), -1) || h.magic != kHelloMagic) { fail = true; break; }
            if (r == 0) { bytes = h.bytes; seq = h.seq; gathered.resize((size_t)bytes * nRanks); }
            else if (h.bytes != bytes || h.seq != seq) { fail = true; break; }
            if (bytes && !ReadAll(byRank[r], gathered.data() + (size_t)r * bytes, bytes, 60000)) fail = true;
        }
        if (fail) break;
        for (uint32_t r = 0; r < nRanks; ++r) {
            ReqHeader h = {kHelloMagic, seq, bytes * nRanks};
            if (!WriteAll(byRank[r], &h, sizeof(h)) || (bytes && !WriteAll(byRank[r], gathered.data(), gathered.size()))) fail = true;
        }
        if (fail) break;
    }
    // A failed or closed connection ends the group: closing every socket makes the
    // surviving ranks' next bootstrap call return an error instead of blocking.
    for (int f : byRank) ::close(f);
}

std::string UdsName(uint64_t uniqueId, int rank)
{
    char buf[96];
    snprintf(buf, sizeof(buf), "hccl-b200-%016llx-%d", (unsigned long long)uniqueId, rank);
    return buf;
}
socklen_t FillUds(struct sockaddr_un* a, const std::string& name)
{
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    a->sun_path[0] = '\0';  // abstract namespace: no file, vanishes with the socket
    memcpy(a->sun_path + 1, name.data(), name.size());
    return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + name.size());
}

// The trust list of HCCL_WHITELIST_FILE: {"host_ip": ["a.b.c.d", ...]} (a "device_ip" array is accepted and unused).
HcclResult LoadWhitelist(const std::string& path, std::set<uint32_t>* out)
{
    std::ifstream in(path);
    if (!in) { HCCL_ERROR("HCCL_WHITELIST_DISABLE=0 but HCCL_WHITELIST_FILE '%s' cannot be read", path.c_str()); return HCCL_E_PARA; }
    std::stringstream ss;
    ss << in.rdbuf();
    JsonValue root;
    std::string err;
    const std::string text = ss.str();
    if (!JsonParser(text).Parse(&root, &err) || root.kind != JsonValue::OBJ) { HCCL_ERROR("HCCL_WHITELIST_FILE '%s': %s", path.c_str(), err.empty() ? "not an object" : err.c_str()); return HCCL_E_PARA; }
    const JsonValue* hosts = root.Get("host_ip");
    if (!hosts || hosts->kind != JsonValue::ARR) { HCCL_ERROR("HCCL_WHITELIST_FILE '%s': no \"host_ip\" array", path.c_str()); return HCCL_E_PARA; }
    for (const JsonValue& v : hosts->arr) {
        struct in_addr a;
        if (v.kind != JsonValue::STR || inet_pton(AF_INET, v.str.c_str(), &a) != 1) { HCCL_ERROR("HCCL_WHITELIST_FILE '%s': '%s' is not a dotted IPv4 address", path.c_str(), v.str.c_str()); return HCCL_E_PARA; }
        out->insert(a.s_addr);
    }
    return HCCL_SUCCESS;
}

}  // namespace

// Which of the interfaces (name order as given) a rule of HCCL_SOCKET_IFNAME selects: -1 when none.  "eth,enp":
// names with one of the prefixes; "=eth0,enp0": exactly these; a leading '^' turns either into an exclusion.
int MatchInterfaceRule(const std::string& rule, const std::vector<std::string>& names)
{
    std::string body = rule;
    bool exclude = false, exact = false;
    if (!body.empty() && body[0] == '^') { exclude = true; body.erase(0, 1); }
    if (!body.empty() && body[0] == '=') { exact = true; body.erase(0, 1); }
    std::vector<std::string> keys;
    std::stringstream ss(body);
    for (std::string k; std::getline(ss, k, ',');)
        if (!k.empty()) keys.push_back(k);
    auto listed = [&](const std::string& n) {
        for (const std::string& k : keys)
            if (exact ? n == k : n.compare(0, k.size(), k) == 0) return true;
        return false;
    };
    if (!exclude) {
        // the first key that matches an interface wins (keys are a preference order)
        for (const std::string& k : keys)
            for (size_t i = 0; i < names.size(); ++i)
                if (exact ? names[i] == k : names[i].compare(0, k.size(), k) == 0) return (int)i;
        return -1;
    }
    for (size_t i = 0; i < names.size(); ++i)
        if (!listed(names[i])) return (int)i;
    return -1;
}

namespace {
// IPv4 address of the interface HCCL_SOCKET_IFNAME selects.  Candidates in the order the reference documents for its
// own default: interfaces other than docker* / lo by name, then docker*, then lo.
HcclResult InterfaceAddress(const std::string& rule, std::string* ip)
{
    struct ifaddrs* list = nullptr;
    if (getifaddrs(&list) != 0) return HCCL_E_SYSCALL;
    std::vector<std::pair<std::string, std::string>> found;
    for (struct ifaddrs* it = list; it; it = it->ifa_next) {
        if (!it->ifa_addr || it->ifa_addr->sa_family != AF_INET || !(it->ifa_flags & IFF_UP)) continue;
        char text[INET_ADDRSTRLEN] = {0};
        inet_ntop(AF_INET, &((struct sockaddr_in*)it->ifa_addr)->sin_addr, text, sizeof(text));
        found.emplace_back(it->ifa_name, text);
    }
    freeifaddrs(list);
    auto klass = [](const std::string& n) { return n == "lo" ? 2 : n.compare(0, 6, "docker") == 0 ? 1 : 0; };
    std::sort(found.begin(), found.end(), [&](const auto& a, const auto& b) { return klass(a.first) != klass(b.first) ? klass(a.first) < klass(b.first) : a.first < b.first; });
    std::vector<std::string> names;
    for (auto& f : found) names.push_back(f.first);
    const int i = MatchInterfaceRule(rule, names);
    if (i < 0) { HCCL_ERROR("HCCL_SOCKET_IFNAME=%s selects none of the %zu interfaces with an IPv4 address", rule.c_str(), names.size()); return HCCL_E_NOT_FOUND; }
    *ip = found[(size_t)i].second;
    HCCL_INFO("rendezvous address %s from interface %s (HCCL_SOCKET_IFNAME=%s)", ip->c_str(), found[(size_t)i].first.c_str(), rule.c_str());
    return HCCL_SUCCESS;
}
}  // namespace

HcclResult BootstrapCreateRootAt(const std::string& ipIn, uint32_t port, uint64_t uniqueId, HcclRootInfo* out)
{
    CHK_PTR_NULL(out);
    const EnvConfig& env = GetEnvConfig();
    if (env.socketIpv6) { HCCL_ERROR("HCCL_SOCKET_FAMILY=AF_INET6: the rendezvous of this library speaks IPv4 only"); return HCCL_E_NOT_SUPPORT; }
    std::shared_ptr<std::set<uint32_t>> allowed;
    if (!env.whitelistDisable) {
        allowed.reset(new std::set<uint32_t>());
        CHK_RET(LoadWhitelist(env.whitelistFile, allowed.get()));
    }
    std::string ip = ipIn.empty() ? "127.0.0.1" : ipIn;
    struct sockaddr_in addr;
    memset(&addr, 0, sizeof(addr));
    addr.sin_family = AF_INET;
    if (inet_pton(AF_INET, ip.c_str(), &addr.sin_addr) != 1) { HCCL_ERROR("bad rendezvous address '%s'", ip.c_str()); return HCCL_E_PARA; }
    // the ports to try: the caller's (a rank table names one), else HCCL_HOST_SOCKET_PORT_RANGE, else whatever is free
    std::vector<uint32_t> ports;
    if (port == 0 && !env.hostPortAuto)
        for (auto& r : env.hostPortRanges)
            for (uint32_t q = r.first; q <= r.second && ports.size() < 4096; ++q) ports.push_back(q);
    if (ports.empty()) ports.push_back(port);
    int fd = -1;
    for (uint32_t q : ports) {
        fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) return HCCL_E_SYSCALL;
        int reuse = 1;
        setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &reuse, sizeof(reuse));
        addr.sin_port = htons((uint16_t)q);
        if (::bind(fd, (struct sockaddr*)&addr, sizeof(addr)) == 0 && ::listen(fd, 256) == 0) break;
        ::close(fd);
        fd = -1;
    }
    if (fd < 0) {
        HCCL_ERROR("cannot listen on %s, ports %u..%u: %s", ip.c_str(), ports.front(), ports.back(), strerror(errno));
        return HCCL_E_TCP_CONNECT;
    }
    socklen_t len = sizeof(addr);
    getsockname(fd, (struct sockaddr*)&addr, &len);
    memset(out, 0, sizeof(*out));
    RootInfoPayload* p = reinterpret_cast<RootInfoPayload*>(out->internal);
    p->magic = kRootInfoMagic;
    p->version = 1;
    snprintf(p->ip, sizeof(p->ip), "%s", ip.c_str());
    p->port = ntohs(addr.sin_port);
    p->uniqueId = uniqueId;
    std::thread(RelayThread, fd, uniqueId, allowed).detach();
    HCCL_INFO("rendezvous endpoint %s:%u id %016llx", p->ip, p->port, (unsigned long long)uniqueId);
    return HCCL_SUCCESS;
}

HcclResult BootstrapCreateRoot(HcclRootInfo* out)
{
    const EnvConfig& env = GetEnvConfig();
    std::random_device rd;
    uint64_t id = ((uint64_t)rd() << 32) ^ rd() ^ ((uint64_t)getpid() << 16) ^
                  (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count();
    // the address: HCCL_IF_IP, else the interface HCCL_SOCKET_IFNAME selects, else the loopback (one box);
    // the port: HCCL_HOST_SOCKET_PORT_RANGE when set (it takes precedence), else HCCL_IF_BASE_PORT, else any
    std::string ip = env.ifIp;
    if (ip.empty() && !env.socketIfname.empty()) CHK_RET(InterfaceAddress(env.socketIfname, &ip));
    const bool ranged = env.hostPortAuto || !env.hostPortRanges.empty();
    return BootstrapCreateRootAt(ip, ranged ? 0 : env.ifBasePort, id, out);
}

Bootstrap::~Bootstrap() { Close(); }

void Bootstrap::Close()
{
    if (tcpFd_ >= 0) { ::close(tcpFd_); tcpFd_ = -1; }
    if (udsFd_ >= 0) { ::close(udsFd_); udsFd_ = -1; }
    for (auto& p : pendingFds_) ::close(p.fd);
    pendingFds_.clear();
}

HcclResult Bootstrap::Connect(const HcclRootInfo& info, int rank, int nRanks, uint32_t timeoutS)
{
    const RootInfoPayload* p = reinterpret_cast<const RootInfoPayload*>(info.internal);
    if (p->magic != kRootInfoMagic) { HCCL_ERROR("root info was not produced by HcclGetRootInfo"); return HCCL_E_PARA; }
    if (nRanks <= 0 || rank < 0 || rank >= nRanks) { HCCL_ERROR("rank %d out of range for %d ranks", rank, nRanks); return HCCL_E_PARA; }
    rank_ = rank; nRanks_ = nRanks; uniqueId_ = p->uniqueId; timeoutS_ = timeoutS ? timeoutS : 120;
    // unix datagram socket for descriptor passing
    udsFd_ = ::socket(AF_UNIX, SOCK_DGRAM, 0);
    if (udsFd_ < 0) return HCCL_E_SYSCALL;
    struct sockaddr_un ua;
    socklen_t ul = FillUds(&ua, UdsName(uniqueId_, rank));
    if (::bind(udsFd_, (struct sockaddr*)&ua, ul) != 0) { HCCL_ERROR("cannot bind descriptor-passing socket: %s", strerror(errno)); return HCCL_E_SYSCALL; }
    // TCP to the relay, retried until the timeout (the root may not be up yet)
    struct sockaddr_in addr;
    memset(&addr, 0, sizeof(addr));
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)p->port);
    if (inet_pton(AF_INET, p->ip, &addr.sin_addr) != 1) return HCCL_E_PARA;
    auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeoutS_);
    for (;;) {
        tcpFd_ = ::socket(AF_INET, SOCK_STREAM, 0);
        if (tcpFd_ < 0) return HCCL_E_SYSCALL;
        if (::connect(tcpFd_, (struct sockaddr*)&addr, sizeof(addr)) == 0) break;
        ::close(tcpFd_);
        tcpFd_ = -1;
        if (std::chrono::steady_clock::now() > deadline) {
            HCCL_ERROR("rank %d: cannot reach rendezvous %s:%u within %u s (HCCL_CONNECT_TIMEOUT)", rank, p->ip, p->port, timeoutS_);
            return HCCL_E_TCP_CONNECT;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    int one = 1;
    setsockopt(tcpFd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    Hello h = {kHelloMagic, (uint32_t)rank, (uint32_t)nRanks, 0, uniqueId_};
    if (!WriteAll(tcpFd_, &h, sizeof(h))) return HCCL_E_TCP_TRANSFER;
    uint32_t ok = 0;
    if (!ReadAll(tcpFd_, &ok, sizeof(ok), (int)timeoutS_ * 1000) || ok != 1) {
        HCCL_ERROR("rank %d: the group of %d ranks did not complete within %u s (a rank never joined?)", rank, nRanks, timeoutS_);
        return HCCL_E_TIMEOUT;
    }
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::AllGather(const void* send, void* recv, size_t bytes)
{
    std::lock_guard<std::mutex> lk(mu_);
    if (tcpFd_ < 0) return HCCL_E_NETWORK;
    if (injectFail_) { injectFail_ = false; ::shutdown(tcpFd_, SHUT_RDWR); return HCCL_E_TCP_TRANSFER; }
    static thread_local uint32_t dummy = 0;
    (void)dummy;
    ReqHeader h = {kHelloMagic, 0, (uint64_t)bytes};
    if (!WriteAll(tcpFd_, &h, sizeof(h)) || (bytes && !WriteAll(tcpFd_, send, bytes))) return HCCL_E_TCP_TRANSFER;
    ReqHeader r;
    if (!ReadAll(tcpFd_, &r, sizeof(r), (int)timeoutS_ * 1000) || r.magic != kHelloMagic || r.bytes != bytes * (uint64_t)nRanks_) {
        HCCL_ERROR("rank %d: rendezvous exchange failed or timed out after %u s (a peer left or mismatched call)", rank_, timeoutS_);
        return HCCL_E_REMOTE;
    }
    if (bytes && !ReadAll(tcpFd_, recv, bytes * (size_t)nRanks_, (int)timeoutS_ * 1000)) return HCCL_E_TCP_TRANSFER;
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::Barrier() { return AllGather(nullptr, nullptr, 0); }

HcclResult Bootstrap::AgreeAll(bool ok, bool* all)
{
    std::vector<uint8_t> v((size_t)nRanks_);
    uint8_t mine = ok ? 1 : 0;
    CHK_RET(AllGather(&mine, v.data(), 1));
    *all = true;
    for (uint8_t x : v) *all = *all && x != 0;
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::SendFd(int peer, int fd)
{
    struct sockaddr_un ua;
    socklen_t ul = FillUds(&ua, UdsName(uniqueId_, peer));
    int32_t payload = rank_;
    struct iovec iov = {&payload, sizeof(payload)};
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    struct msghdr msg;
    memset(&msg, 0, sizeof(msg));
    msg.msg_name = &ua;
    msg.msg_namelen = ul;
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
    auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeoutS_);
    for (;;) {
        if (::sendmsg(udsFd_, &msg, 0) >= 0) return HCCL_SUCCESS;
        if ((errno == ECONNREFUSED || errno == ENOENT || errno == EAGAIN || errno == ENOBUFS) &&
            std::chrono::steady_clock::now() < deadline) {
            std::this_thread::sleep_for(std::chrono::milliseconds(5));
            continue;
        }
        HCCL_ERROR("rank %d: passing a descriptor to rank %d failed: %s", rank_, peer, strerror(errno));
        return HCCL_E_SYSCALL;
    }
}

HcclResult Bootstrap::RecvFd(int peer, int* fd)
{
    for (auto it = pendingFds_.begin(); it != pendingFds_.end(); ++it) {
        if (it->from == peer) { *fd = it->fd; pendingFds_.erase(it); return HCCL_SUCCESS; }
    }
    for (;;) {
        struct pollfd pf = {udsFd_, POLLIN, 0};
        int pr = ::poll(&pf, 1, (int)timeoutS_ * 1000);
        if (pr == 0) { HCCL_ERROR("rank %d: no descriptor from rank %d within %u s", rank_, peer, timeoutS_); return HCCL_E_TIMEOUT; }
        if (pr < 0) { if (errno == EINTR) continue; return HCCL_E_SYSCALL; }
        int32_t payload = -1;
        struct iovec iov = {&payload, sizeof(payload)};
        char ctrl[CMSG_SPACE(sizeof(int))];
        struct msghdr msg;
        memset(&msg, 0, sizeof(msg));
        msg.msg_iov = &iov;
        msg.msg_iovlen = 1;
        msg.msg_control = ctrl;
        msg.msg_controllen = sizeof(ctrl);
        ssize_t r = ::recvmsg(udsFd_, &msg, 0);
        if (r < 0) { if (errno == EINTR) continue; return HCCL_E_SYSCALL; }
        struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
        if (!c || c->cmsg_type != SCM_RIGHTS) continue;
        int got;
        memcpy(&got, CMSG_DATA(c), sizeof(int));
        if (payload == peer) { *fd = got; return HCCL_SUCCESS; }
        pendingFds_.push_back({payload, got});
    }
}

}  // namespace hccl
