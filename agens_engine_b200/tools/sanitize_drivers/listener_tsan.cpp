// The HTTP listener and the callback backend under ThreadSanitizer: twelve client threads (socket and in-process
// requests, streamed and plain, some dropped early) while engine-side threads push tokens.  Built and run by
// tools/sanitize.py (tsan-listener) together with the server sources; argv[1] is a tokenizer.json.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>
extern "C" {
typedef void (*GenerateFn)(void*, long long, const int*, int, const char*, const char*);
void* b2h_server_new(const char*, char*, int);
void b2h_server_free(void*);
void b2h_server_use_callback(void*, GenerateFn, void*, int);
int b2h_stream_push(void*, long long, const int*, int, int, const char*);
int b2h_stream_cancelled(void*, long long);
char* b2h_server_handle(void*, const char*, const char*, const char*, const char*, int*);
int b2h_server_start(void*, const char*, int);
void b2h_server_stop(void*);
void b2h_server_set_metrics(void*, const char*);

}
static void b2h_free_str(char* p) { free(p); }
static void* g_srv;
static std::atomic<long> g_done{0}, g_cancel{0};
static void gen(void*, long long rid, const int*, int n, const char*, const char*) {
  std::thread([rid, n]() {
    for (int i = 0; i < 12; ++i) {
      int ids[2] = {65 + (int)((rid + i) % 26), 97 + i};
      if (b2h_stream_push(g_srv, rid, ids, 2, 0, nullptr)) { ++g_cancel; break; }
      if (i % 4 == 0) std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    b2h_stream_push(g_srv, rid, nullptr, 0, 1, nullptr);
    ++g_done;
  }).detach();
}
static std::string http(int port, const std::string& req, bool drop_early) {
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  sockaddr_in a{}; a.sin_family = AF_INET; a.sin_port = htons((uint16_t)port); inet_pton(AF_INET, "127.0.0.1", &a.sin_addr);
  if (connect(fd, (sockaddr*)&a, sizeof a) != 0) { close(fd); return ""; }
  send(fd, req.data(), req.size(), MSG_NOSIGNAL);
  std::string out; char buf[4096]; ssize_t n;
  while ((n = recv(fd, buf, sizeof buf, 0)) > 0) { out.append(buf, (size_t)n); if (drop_early && out.size() > 200) break; }
  close(fd);
  return out;
}
int main(int argc, char** argv) {
  char err[256];
  if (argc < 2) { printf("usage: listener_tsan tokenizer.json\n"); return 2; }
  const std::string cfg = std::string("{\"tokenizer_json\": \"") + argv[1] + "\", \"model_name\": \"m\", \"eos_token_ids\": []}";
  g_srv = b2h_server_new(cfg.c_str(), err, 256);
  if (!g_srv) { printf("no server: %s\n", err); return 1; }
  b2h_server_use_callback(g_srv, gen, nullptr, 4096);
  int port = b2h_server_start(g_srv, "127.0.0.1", 0);
  std::vector<std::thread> th;
  std::atomic<long> ok{0};
  for (int t = 0; t < 12; ++t)
    th.emplace_back([&, t]() {
      for (int i = 0; i < 40; ++i) {
        const bool stream = (i + t) % 2, chat = i % 3 != 0;
        std::string body = chat ? std::string("{\"messages\": [{\"role\": \"user\", \"content\": \"hi\"}], \"max_tokens\": 30, \"stream\": ") + (stream ? "true" : "false") + "}"
                                : std::string("{\"prompt\": \"abc\", \"max_tokens\": 30, \"stream\": ") + (stream ? "true" : "false") + "}";
        if (t % 4 == 3) {          // in-process handle path and metrics
          int st = 0; char* r = b2h_server_handle(g_srv, "POST", chat ? "/v1/chat/completions" : "/v1/completions", "", body.c_str(), &st); if (st == 200) ++ok; b2h_free_str(r);
          r = b2h_server_handle(g_srv, "GET", "/metrics", "", "", &st); b2h_free_str(r);
          b2h_server_set_metrics(g_srv, "x 1\n");
        } else {
          std::string req = std::string("POST ") + (chat ? "/v1/chat/completions" : "/v1/completions") + " HTTP/1.1\r\nContent-Length: " + std::to_string(body.size()) + "\r\n\r\n" + body;
          std::string r = http(port, req, stream && i % 5 == 0);
          if (r.find("200 OK") != std::string::npos) ++ok;
        }
      }
    });
  for (auto& x : th) x.join();
  std::this_thread::sleep_for(std::chrono::milliseconds(500));
  b2h_server_stop(g_srv);
  printf("ok %ld done %ld cancelled %ld\n", ok.load(), g_done.load(), g_cancel.load());
  return ok.load() == 480 ? 0 : 1;
}
