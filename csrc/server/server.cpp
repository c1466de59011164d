// OpenAI-compatible HTTP front end: /health, /health_generate, /metrics, /v1/models, /v1/models/{name},
// /v1/chat/completions, /v1/completions with SSE streaming, stop strings, incremental detokenisation, reasoning and
// tool-call parsing, usage accounting and cancellation when the client goes away.
//
// Reference: crates/agens-server/src/{server.rs:90-99, openai.rs:244-385 & 742-835, engine.rs, sampling.rs:104-205,
// backend.rs:1-64}.  The engine is reached through a Backend: generate() returns at once and the engine pushes each
// step's accepted ids (one or several with speculation) into the request's stream; the server owns stop strings,
// text, parsing and usage.  MockBackend replays a scripted id list in fixed steps, as the reference's test backend.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cctype>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <deque>
#include <fstream>
#include <functional>
#include <memory>
#include <mutex>
#include <random>
#include <sstream>
#include <system_error>
#include <thread>

#include "text.hpp"

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace b2 {

// ------------------------------------------------------------------------------------------------ backend
struct TokenStream {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::vector<int>> q;
  bool finished = false, cancelled = false;
  std::string error;
  void push(const int* ids, int n, bool fin, const char* err = nullptr) {
    std::lock_guard<std::mutex> l(mu);
    if (n > 0) q.emplace_back(ids, ids + n);
    if (fin) finished = true;
    if (err) { error = err; finished = true; }
    cv.notify_all();
  }
  // false when the stream is finished and drained
  bool pop(std::vector<int>& out) {
    std::unique_lock<std::mutex> l(mu);
    cv.wait(l, [&] { return !q.empty() || finished; });
    if (q.empty()) return false;
    out = std::move(q.front());
    q.pop_front();
    return true;
  }
  void cancel() { std::lock_guard<std::mutex> l(mu); cancelled = true; }
  bool is_cancelled() { std::lock_guard<std::mutex> l(mu); return cancelled; }
};

struct GenRequest { long long id; std::vector<int> prompt; Json sampling; std::string session_id; Json images; };

class Backend {
 public:
  virtual ~Backend() {}
  virtual void generate(const GenRequest& r, std::shared_ptr<TokenStream> s) = 0;
  virtual bool supports_images() const { return false; }
  virtual int context_length() const { return 262144; }
};

class MockBackend : public Backend {
 public:
  std::vector<int> script;
  int step = 1;
  bool images = false;
  std::mutex mu;
  std::vector<GenRequest> calls;
  void generate(const GenRequest& r, std::shared_ptr<TokenStream> s) override {
    { std::lock_guard<std::mutex> l(mu); calls.push_back(r); }
    const long long maxn = r.sampling.get_int("max_new_tokens", 1 << 30);
    std::vector<int> out = script;
    if ((long long)out.size() > maxn) out.resize((size_t)maxn);
    std::thread([out, s, st = step]() {
      for (size_t i = 0; i < out.size(); i += st) {
        if (s->is_cancelled()) break;
        const int n = (int)std::min<size_t>(st, out.size() - i);
        s->push(out.data() + i, n, false);
      }
      s->push(nullptr, 0, true);
    }).detach();
  }
  bool supports_images() const override { return images; }
};

typedef void (*GenerateFn)(void* user, long long req_id, const int* prompt, int n_prompt, const char* sampling_json, const char* session_id);

class CallbackBackend : public Backend {
 public:
  GenerateFn fn = nullptr;
  void* user = nullptr;
  int ctx = 262144;
  bool images = false;
  bool supports_images() const override { return images; }
  std::mutex mu;
  std::map<long long, std::shared_ptr<TokenStream>> streams;
  void generate(const GenRequest& r, std::shared_ptr<TokenStream> s) override {
    { std::lock_guard<std::mutex> l(mu); streams[r.id] = s; }
    fn(user, r.id, r.prompt.data(), (int)r.prompt.size(), r.sampling.dump().c_str(), r.session_id.c_str());
  }
  std::shared_ptr<TokenStream> find(long long id) { std::lock_guard<std::mutex> l(mu); auto it = streams.find(id); return it == streams.end() ? nullptr : it->second; }
  void drop(long long id) { std::lock_guard<std::mutex> l(mu); streams.erase(id); }
  int context_length() const override { return ctx; }
};

// ------------------------------------------------------------------------------------------------ server state
struct HttpResponse { int status = 200; std::string content_type = "application/json", body; bool sse = false; };

// Markers of the model's output language: the think block and the tool-call wrapper.  Two families are known: the
// ChatML one and the reference model's (<|think|> ... <|/think|>, <|call|> ... <|/call|>); the checkpoint's chat template
// tells which (it writes the markers itself).
struct TagSet { std::string think_open = "<think>", think_close = "</think>", call_open = "<tool_call>", call_close = "</tool_call>"; };

struct Server {
  TagSet tags;
  std::vector<int> think_close_ids;        // token ids of the closing think tag (reasoning token count)
  Tokenizer tok;
  bool has_tok = false;
  std::string model_name = "b200-engine";
  Json gen_defaults = Json::object();      // generation_config.json: temperature, top_k, top_p
  std::vector<int> eos_ids;
  long long max_tokens_default = 32768;
  std::string chat_template;               // Jinja source from tokenizer_config.json; empty = the built-in ChatML renderer
  std::string bos_token, eos_token;
  std::shared_ptr<Backend> backend;
  std::atomic<long long> next_req{1}, n_requests{0}, n_prompt_tokens{0}, n_completion_tokens{0}, n_errors{0};
  std::mutex extra_mu;
  std::string extra_metrics;               // engine-side gauges (scheduler steps, step times, KV pages), set by the engine
  std::atomic<int> listen_fd{-1};
  std::thread accept_thread;
  std::atomic<bool> stopping{false};
  std::atomic<int> live_connections{0};      // connection threads that still use this object
};

static std::string hex_id(int n) {
  static std::mt19937_64 rng{std::random_device{}()};
  static std::mutex mu;
  std::lock_guard<std::mutex> l(mu);
  static const char* d = "0123456789abcdef";
  std::string s;
  for (int i = 0; i < n; ++i) s.push_back(d[rng() & 15]);
  return s;
}

// Error bodies have the reference server's shape (crates/agens-server/src/openai.rs:17-42): a flat object; requests that
// fail validation are "BadRequestError", those refused while the conversation is converted (template errors, bad
// tool-call arguments in the history) "BadRequest".
static HttpResponse error_response(int status, const std::string& msg, const std::string& type = "BadRequestError") {
  Json o = Json::object();
  o.set("object", "error"); o.set("message", msg); o.set("type", type); o.set("param", Json()); o.set("code", status);
  HttpResponse r; r.status = status; r.body = o.dump();
  return r;
}

// Sampling parameters of a request: defaults, then the request's fields, validated (sampling.rs:132-205).
static std::string build_sampling(const Server& sv, const Json& body, bool chat, Json& out) {
  out = Json::object();
  double temperature = chat ? sv.gen_defaults.get_double("temperature", 1.0) : 1.0;
  double top_p = chat ? sv.gen_defaults.get_double("top_p", 1.0) : 1.0;
  long long top_k = chat ? sv.gen_defaults.get_int("top_k", -1) : -1;
  auto num = [&](const char* k, double& v) -> bool { if (auto p = body.find(k); p && !p->is_null()) { if (!p->is_number()) return false; v = p->as_double(); } return true; };
  double min_p = 0, pres = 0, freq = 0, rep = 1;
  if (!num("temperature", temperature) || !num("top_p", top_p) || !num("min_p", min_p) || !num("presence_penalty", pres) ||
      !num("frequency_penalty", freq) || !num("repetition_penalty", rep)) return "sampling parameters must be numbers";
  if (auto p = body.find("top_k"); p && p->is_number()) top_k = p->as_int();
  if (temperature < 0) return "temperature must be non-negative, got " + Json(temperature).dump() + ".";
  if (top_p <= 0 || top_p > 1) return "top_p must be in (0, 1], got " + Json(top_p).dump() + ".";
  if (min_p < 0 || min_p > 1) return "min_p must be in [0, 1], got " + Json(min_p).dump() + ".";
  if (top_k < -1 || top_k == 0) return "top_k must be -1 (disable) or at least 1, got " + std::to_string(top_k) + ".";
  if (freq < -2 || freq > 2) return "frequency_penalty must be in [-2, 2], got " + Json(freq).dump() + ".";
  if (pres < -2 || pres > 2) return "presence_penalty must be in [-2, 2], got " + Json(pres).dump() + ".";
  if (rep <= 0 || rep > 2) return "repetition_penalty must be in (0, 2], got " + Json(rep).dump() + ".";
  if (temperature < 1e-6) { temperature = 1.0; top_k = 1; }     // greedy is expressed as top_k = 1
  long long max_new = sv.max_tokens_default;
  if (auto p = body.find("max_completion_tokens"); p && p->is_number()) max_new = p->as_int();
  else if (auto q = body.find("max_tokens"); q && q->is_number()) max_new = q->as_int();
  if (max_new < 0) return "max_new_tokens must be at least 0, got " + std::to_string(max_new) + ".";
  const long long min_new = body.get_int("min_tokens", 0);
  if (min_new > max_new) return "min_tokens must not exceed max_tokens";
  out.set("temperature", temperature); out.set("top_p", top_p); out.set("top_k", top_k); out.set("min_p", min_p);
  out.set("presence_penalty", pres); out.set("frequency_penalty", freq); out.set("repetition_penalty", rep);
  out.set("max_new_tokens", max_new); out.set("min_new_tokens", min_new);
  if (auto p = body.find("seed"); p && p->is_number()) out.set("seed", p->as_int());
  if (auto p = body.find("logit_bias"); p && p->is_object()) out.set("logit_bias", *p);
  Json stops = Json::array();
  if (!body.get_bool("ignore_eos", false)) for (int e : sv.eos_ids) stops.push_back(e);
  if (auto p = body.find("stop_token_ids"); p && p->is_array()) for (auto& v : p->items()) stops.push_back(v.as_int());
  out.set("stop_token_ids", stops);
  out.set("ignore_eos", body.get_bool("ignore_eos", false));
  // ids beyond the tokenizer (padding rows of the embedding) are never produced
  if (sv.has_tok) out.set("vocab_valid", sv.tok.size());
  return "";
}

static std::string reject_unsupported(const Json& body, bool chat) {
  for (const char* k : {"response_format", "regex", "ebnf", "json_schema", "stop_regex", "input_ids", "custom_logit_processor"})
    if (auto p = body.find(k); p && !p->is_null()) return std::string(k) + " is not supported";
  if (body.get_int("n", 1) > 1) return "n > 1 is not supported";
  if (auto p = body.find("logprobs"); p && ((p->is_bool() && p->as_bool()) || (p->is_number() && p->as_int() > 0))) return "logprobs is not supported";
  if (!chat) {
    if (body.get_bool("echo", false)) return "echo is not supported";
    if (auto p = body.find("suffix"); p && !p->is_null()) return "suffix is not supported";
  }
  return "";
}

// Earliest position at which any stop string begins, or npos; `hold` receives how many trailing bytes might still
// grow into a stop string and must not be emitted yet.
static size_t find_stop(const std::string& text, const std::vector<std::string>& stops, size_t& hold) {
  size_t best = std::string::npos;
  hold = 0;
  for (auto& s : stops) {
    if (s.empty()) continue;
    const size_t p = text.find(s);
    if (p != std::string::npos) best = std::min(best, p);
    const size_t m = std::min(text.size(), s.size() - 1);
    for (size_t k = m; k > 0; --k) if (text.compare(text.size() - k, k, s, 0, k) == 0) { hold = std::max(hold, k); break; }
  }
  return best;
}

struct Emit { std::function<void(const std::string&)> write; std::function<bool()> alive; };

// Runs one generation to completion.  Streaming responses are written through `emit` as SSE events; the complete
// response body (JSON or the concatenated event stream) is returned as well.
static void normalize_schema_types(Json& sc);
// The request's tools as the output parsers use them: none under tool_choice "none", parameter schemas with their
// type names in JSON-schema form.
static Json request_tools(const Json& body) {
  if (!(body.find("tools") && body.at("tools").is_array()) || body.get_string("tool_choice", "auto") == "none") return Json::array();
  Json tools = body.at("tools");
  for (auto& t : tools.items())
    if (t.is_object())
      for (auto& kv : t.members())
        if (kv.first == "function" && kv.second.is_object())
          for (auto& fk : kv.second.members()) if (fk.first == "parameters") normalize_schema_types(fk.second);
  return tools;
}

static HttpResponse run_generation(Server& sv, const Json& body, bool chat, const std::vector<int>& prompt_ids, const Json& sampling,
                                   bool starts_in_reasoning, const std::string& session_id, Emit* emit, bool thinking = false) {
  const bool stream = body.get_bool("stream", false);
  const Json* so = body.find("stream_options");
  const bool include_usage = so && so->is_object() && so->get_bool("include_usage", false);
  const bool continuous_usage = include_usage && so->get_bool("continuous_usage_stats", false);
  const bool separate_reasoning = body.get_bool("separate_reasoning", true);
  const bool stream_reasoning = body.get_bool("stream_reasoning", true);
  const bool skip_special = body.get_bool("skip_special_tokens", true);
  const bool no_stop_trim = body.get_bool("no_stop_trim", false);
  const Json tools = request_tools(body);
  const bool tools_active = chat && tools.size() > 0;
  const TagSet& tg = sv.tags;
  std::vector<std::string> stops;
  if (auto p = body.find("stop")) { if (p->is_string()) stops.push_back(p->as_string()); else if (p->is_array()) for (auto& s : p->items()) if (s.is_string()) stops.push_back(s.as_string()); }
  std::vector<int> stop_ids;
  for (auto& v : sampling.at("stop_token_ids").items()) stop_ids.push_back((int)v.as_int());
  const long long max_new = sampling.get_int("max_new_tokens", sv.max_tokens_default);
  const long long min_new = sampling.get_int("min_new_tokens", 0);

  GenRequest req;
  req.id = sv.next_req++;
  req.prompt = prompt_ids;
  req.sampling = sampling;
  req.session_id = session_id;
  auto ts = std::make_shared<TokenStream>();
  sv.n_requests++;
  sv.n_prompt_tokens += (long long)prompt_ids.size();
  if (max_new > 0) sv.backend->generate(req, ts); else ts->push(nullptr, 0, true);

  // The wire format is the reference server's (crates/agens-server/src/openai.rs:848-1180): a client-chosen "rid" is the
  // response id; every choice carries logprobs / matched_stop; usage counts the tokens through the stop token and the
  // reasoning tokens through the closing think tag.
  const std::string id = body.find("rid") && body.at("rid").is_string() ? body.at("rid").as_string()
                                                                          : (chat ? "chatcmpl-" : "cmpl-") + hex_id(24);
  const long long created = (long long)std::time(nullptr);
  Detokenizer detok(&sv.tok, skip_special);
  ReasoningParser rp(starts_in_reasoning, stream_reasoning, tg.think_open, tg.think_close);
  ToolStreamParser tp(tools, tg.call_open, tg.call_close);
  if (tg.think_open != "<think>") rp.keep_newlines_after_close(true);
  if (tg.call_open != "<tool_call>" && tools_active) { rp.set_interrupt(tg.call_open); tp.content_before_calls_only(true); }
  // streamed calls of the <function=...> family go out piece by piece (name, then the arguments as parameters complete)
  ToolDeltaParser dp(tools, tg.call_open, tg.call_close);
  const bool call_deltas = stream && tools_active && tg.call_open != "<tool_call>";
  std::string text_all, content_all, reasoning_all, sse_all, pending_text;
  std::vector<ToolCall> calls;
  long long n_out = 0, n_reasoning_tokens = 0;
  std::string finish = "length";
  Json matched = Json();                         // stop token id, stop string, or null
  // reasoning tokens: every token of a request with thinking on, through the closing think tag when one comes
  // (with the built-in ChatML renderer the model opens its think block itself, if at all: counted from the text below)
  bool count_reasoning = !sv.chat_template.empty() && (thinking || starts_in_reasoning) && !sv.think_close_ids.empty();
  bool force_nonempty = false;                   // chat_template_kwargs.force_nonempty_content: reasoning alone becomes the content
  if (auto k = body.find("chat_template_kwargs"); k && k->is_object()) force_nonempty = k->get_bool("force_nonempty_content", false);
  std::string whole;                             // non-streaming: the text is parsed once, when it is complete
  std::string final_text;                        // streamed completions: text of the last step
  size_t think_match = 0;

  auto usage_json = [&]() {
    Json u = Json::object();
    u.set("prompt_tokens", (long long)prompt_ids.size()); u.set("total_tokens", (long long)prompt_ids.size() + n_out);
    u.set("completion_tokens", n_out); u.set("prompt_tokens_details", Json()); u.set("reasoning_tokens", n_reasoning_tokens);
    return u;
  };
  auto send = [&](const Json& chunk) {
    const std::string ev = "data: " + chunk.dump() + "\n\n";
    sse_all += ev;
    if (emit) emit->write(ev);
  };
  auto base_chunk = [&]() {
    Json c = Json::object();
    c.set("id", id); c.set("object", chat ? "chat.completion.chunk" : "text_completion"); c.set("created", created); c.set("model", sv.model_name);
    return c;
  };
  auto wrap = [&](Json choice, bool with_usage_key) {
    Json c = base_chunk(), arr = Json::array();
    arr.push_back(std::move(choice));
    c.set("choices", arr);
    if (continuous_usage) c.set("usage", usage_json());
    else if (with_usage_key) c.set("usage", Json());
    return c;
  };
  auto choice_of = [&](Json delta) {
    Json ch = Json::object();
    ch.set("index", 0); ch.set("delta", std::move(delta)); ch.set("logprobs", Json()); ch.set("finish_reason", Json()); ch.set("matched_stop", Json());
    return ch;
  };
  // chat deltas come in the reference's two shapes: the short one (reasoning / plain content) and, once the request has
  // tools, the long one with every field present
  auto reasoning_chunk = [&](const std::string& r) { Json d = Json::object(); d.set("reasoning_content", r); return wrap(choice_of(d), false); };
  auto content_chunk = [&](const std::string& c) {
    Json d = Json::object();
    if (tools_active) { d.set("role", Json()); d.set("content", c); d.set("reasoning_content", Json()); d.set("tool_calls", Json()); }
    else { d.set("reasoning_content", Json()); d.set("content", c); }
    return wrap(choice_of(d), tools_active);
  };
  auto call_chunk = [&](const Json& id_, long long index, const Json& name, const std::string& args) {
    Json fn = Json::object(), tc = Json::object(), arr = Json::array(), d = Json::object();
    fn.set("name", name); fn.set("arguments", args);
    tc.set("id", id_); tc.set("index", index); tc.set("type", "function"); tc.set("function", fn);
    arr.push_back(tc);
    d.set("role", Json()); d.set("content", Json()); d.set("reasoning_content", Json()); d.set("tool_calls", arr);
    return wrap(choice_of(d), true);
  };
  auto text_chunk = [&](const std::string& t, const Json& fin, const Json& ms) {      // /v1/completions
    Json ch = Json::object();
    ch.set("index", 0); ch.set("text", t); ch.set("logprobs", Json()); ch.set("finish_reason", fin); ch.set("matched_stop", ms);
    Json c = base_chunk(), arr = Json::array();
    arr.push_back(ch); c.set("choices", arr);
    c.set("usage", continuous_usage ? usage_json() : Json());
    return c;
  };
  if (stream && chat) {
    Json d = Json::object();
    d.set("reasoning_content", Json()); d.set("role", "assistant"); d.set("content", "");
    Json c = base_chunk(), arr = Json::array();
    arr.push_back(choice_of(d)); c.set("choices", arr);
    send(c);
  }
  // text -> (reasoning, content, tool calls) -> client
  auto process_text = [&](const std::string& piece, bool last) {
    ReasoningParser::Out ro;
    if (chat && separate_reasoning) { ro = rp.push(piece); if (last) { auto f = rp.finish(); ro.content += f.content; ro.reasoning += f.reasoning; } }
    else ro.content = piece;
    reasoning_all += ro.reasoning;
    if (call_deltas) {
      if (!ro.reasoning.empty()) send(reasoning_chunk(ro.reasoning));
      const std::vector<ToolDelta> ds = dp.push(ro.content);
      std::string plain;                          // the content of one step goes out first, then the call pieces in order
      for (auto& d : ds) if (d.kind == ToolDelta::Content) plain += d.text;
      if (!plain.empty()) { content_all += plain; send(content_chunk(plain)); }
      for (auto& d : ds) {
        if (d.kind == ToolDelta::Content) continue;
        if (d.kind == ToolDelta::Start) { send(call_chunk(Json("call_" + hex_id(24)), d.index, Json(d.text), "")); calls.push_back(ToolCall{d.text, ""}); }
        else { send(call_chunk(Json(), d.index, Json(), d.text)); if (d.index >= 0 && d.index < (int)calls.size()) calls[d.index].arguments_json += d.text; }
      }
      return;
    }
    ToolParse t;
    if (tools_active) { t = tp.push(ro.content); if (last) { auto f = tp.finish(); t.content += f.content; for (auto& c : f.calls) t.calls.push_back(c); } }
    else t.content = ro.content;
    content_all += t.content;
    if (!stream) { for (auto& c : t.calls) calls.push_back(c); return; }
    if (!ro.reasoning.empty()) send(reasoning_chunk(ro.reasoning));
    if (!t.content.empty()) send(chat ? content_chunk(t.content) : text_chunk(t.content, Json(), Json()));
    for (auto& c : t.calls) {
      // a call goes out as its header (id, name, empty arguments) followed by its arguments
      const long long index = (long long)calls.size();
      send(call_chunk(Json("call_" + hex_id(24)), index, Json(c.name), ""));
      send(call_chunk(Json(), index, Json(), c.arguments_json));
      calls.push_back(c);
    }
  };

  std::vector<int> step_ids;
  bool done = false;
  while (!done && ts->pop(step_ids)) {
    std::string step_text;                        // one engine step = one event per kind of text
    size_t step_hold = 0;
    // reasoning tokens are counted per engine step, before the step is cut at a stop (the reference counts that way):
    // tokens through the closing think tag
    for (size_t i = 0; i < step_ids.size() && count_reasoning && n_out + (long long)i < max_new; ++i) {
      const int tkn = step_ids[i];
      ++n_reasoning_tokens;
      think_match = tkn == sv.think_close_ids[think_match] ? think_match + 1 : (tkn == sv.think_close_ids[0] ? 1 : 0);
      if (think_match == sv.think_close_ids.size()) count_reasoning = false;
    }
    for (int tkn : step_ids) {
      if (n_out >= max_new) { done = true; break; }
      ++n_out;
      const bool is_stop_id = std::find(stop_ids.begin(), stop_ids.end(), tkn) != stop_ids.end() && n_out > min_new;
      if (is_stop_id) { finish = "stop"; matched = Json((long long)tkn); done = true; break; }
      std::string piece = detok.push({tkn});
      text_all += piece;
      pending_text += piece;
      size_t hold = 0;
      const size_t sp = find_stop(pending_text, stops, hold);
      if (sp != std::string::npos) {
        std::string upto = pending_text.substr(0, sp);
        for (auto& s : stops) if (!s.empty() && pending_text.compare(sp, s.size(), s) == 0) { matched = Json(s); if (no_stop_trim) upto += s; break; }
        step_text += upto;
        pending_text.clear();
        finish = "stop"; done = true; break;
      }
      step_hold = hold;
      if (n_out >= max_new) { done = true; break; }
    }
    // once per engine step: while the end of the text could still grow into a stop string nothing of it goes out
    if (step_hold == 0 || finish == "stop") { step_text += pending_text; pending_text.clear(); }     // (a matched stop string left nothing pending)
    if (!stream) whole += step_text;
    else if (!chat) {
      // /v1/completions: one event per engine step; the step that ends the request carries its text and the finish reason
      content_all += step_text;
      if (done) final_text = step_text;
      else if (!step_text.empty()) send(text_chunk(step_text, Json(), Json()));
    } else if (!step_text.empty()) process_text(step_text, false);
    if (emit && !emit->alive()) { ts->cancel(); done = true; finish = "abort"; }
  }
  ts->cancel();     // the engine stops at its next step once the receiver is gone
  if (auto cb = dynamic_cast<CallbackBackend*>(sv.backend.get())) cb->drop(req.id);
  if (!ts->error.empty()) { sv.n_errors++; return error_response(500, ts->error, "InternalServerError"); }
  { std::string tail = detok.finish(); if (finish != "stop") pending_text += tail; }
  if (!stream) {
    whole += finish == "stop" ? std::string() : pending_text;
    // with the whole text in hand a think block that closes later keeps a call marker inside it as reasoning
    if (whole.find(tg.think_close) != std::string::npos) rp.set_interrupt("");
    process_text(whole, true);
  } else if (!chat) {
    if (finish != "stop") { final_text += pending_text; content_all += pending_text; }
  } else process_text(finish == "stop" ? std::string() : pending_text, true);
  if (force_nonempty && chat && content_all.empty() && calls.empty() && !reasoning_all.empty()) {
    if (stream) send(content_chunk(reasoning_all));
    content_all = reasoning_all;
    reasoning_all.clear();
  }
  if (sv.chat_template.empty() && chat && !reasoning_all.empty() && sv.has_tok)
    n_reasoning_tokens = std::min<long long>(n_out, (long long)sv.tok.encode(tg.think_open + reasoning_all).size() + (long long)sv.think_close_ids.size());
  // a stop token after at least one call reads as "tool_calls"; the complete response then reports no matched stop
  const bool by_calls = !calls.empty() && finish == "stop" && matched.is_int();
  sv.n_completion_tokens += n_out;

  HttpResponse resp;
  if (stream) {
    if (chat) {
      Json d = Json::object(), ch = Json::object();
      d.set("reasoning_content", Json());
      ch.set("index", 0); ch.set("delta", d); ch.set("logprobs", Json()); ch.set("finish_reason", by_calls ? "tool_calls" : finish); ch.set("matched_stop", matched);
      Json c = base_chunk(), arr = Json::array();
      arr.push_back(ch); c.set("choices", arr);
      send(c);
    } else send(text_chunk(final_text, Json(finish), matched));
    if (include_usage) {
      Json c = base_chunk(), u = usage_json();
      if (!chat) {                                // the completions usage event leaves absent details out
        Json v = Json::object();
        for (auto& kv : u.members()) if (!kv.second.is_null()) v.set(kv.first, kv.second);
        u = v;
      }
      c.set("choices", Json::array()); c.set("usage", u); send(c);
    }
    sse_all += "data: [DONE]\n\n";
    if (emit) emit->write("data: [DONE]\n\n");
    resp.sse = true; resp.content_type = "text/event-stream"; resp.body = sse_all;
    return resp;
  }
  Json o = Json::object(), ch = Json::object();
  o.set("id", id); o.set("object", chat ? "chat.completion" : "text_completion"); o.set("created", created); o.set("model", sv.model_name);
  ch.set("index", 0);
  if (chat) {
    Json m = Json::object();
    m.set("role", "assistant");
    m.set("content", content_all);
    m.set("reasoning_content", reasoning_all.empty() ? Json() : Json(reasoning_all));
    if (!calls.empty()) {
      Json arr = Json::array();
      long long index = 0;
      for (auto& c : calls) {
        Json tc = Json::object(), fn = Json::object();
        tc.set("id", "call_" + hex_id(24)); tc.set("index", index++); tc.set("type", "function");
        fn.set("name", c.name); fn.set("arguments", c.arguments_json);
        tc.set("function", fn); arr.push_back(tc);
      }
      m.set("tool_calls", arr);
    } else m.set("tool_calls", Json());
    ch.set("message", m);
  } else ch.set("text", content_all);
  ch.set("logprobs", Json());
  ch.set("finish_reason", by_calls ? "tool_calls" : finish);
  ch.set("matched_stop", by_calls ? Json() : matched);
  Json arr = Json::array(); arr.push_back(ch);
  o.set("choices", arr); o.set("usage", usage_json());
  Json meta = Json::object(); meta.set("weight_version", "default"); o.set("metadata", meta);
  resp.body = o.dump();
  return resp;
}

// Tool parameter schemas may carry database / ORM style type names ("varchar(255)", "int", "list[str]", "map");
// the template (and the typed argument conversion) sees the JSON-schema name instead
// (crates/agens-server/src/toolcall.rs:241-375).  Rules: a standard name stays; otherwise the text before "(" is
// trimmed and lower-cased and looked up: exact aliases first, then family prefixes followed by a digit or bracket.
static std::string schema_type_name(const std::string& raw) {
  static const char* kStd[] = {"null", "boolean", "object", "array", "number", "string", "integer"};
  for (auto t : kStd) if (raw == t) return raw;
  std::string base = raw.substr(0, raw.find('('));
  size_t a = 0, b = base.size();
  while (a < b && std::isspace((unsigned char)base[a])) ++a;
  while (b > a && std::isspace((unsigned char)base[b - 1])) --b;
  base = base.substr(a, b - a);
  for (auto& c : base) c = (char)std::tolower((unsigned char)c);
  for (auto t : kStd) if (base == t) return base;
  struct Family { const char* target; std::vector<const char*> exact, prefix; };
  static const std::vector<Family> kFamilies = {
      {"string", {"str", "text", "varchar", "char", "enum", "uuid", "date", "datetime", "time", "timestamp", "binary", "blob", "bytea", "bytes", "varbinary"}, {}},
      {"boolean", {"bool"}, {}},
      {"integer", {"bigint", "smallint", "tinyint"}, {"int", "uint", "long", "short", "unsigned"}},
      {"number", {"double", "decimal", "real", "numeric"}, {"num", "float"}},
      {"array", {"arr", "tuple", "set"}, {"list"}},
      {"object", {"map"}, {"dict"}},
  };
  for (auto& f : kFamilies) for (auto e : f.exact) if (base == e) return f.target;
  // prefixes in the order integer, number, array, object; within a family in the order listed
  for (auto& f : kFamilies)
    for (auto p : f.prefix) {
      const size_t n = std::strlen(p);
      if (base == p) return f.target;
      if (base.size() > n && base.compare(0, n, p) == 0 && std::strchr("0123456789[<( \t", base[n])) return f.target;
    }
  return raw;
}

static void normalize_schema_types(Json& sc) {
  if (sc.is_array()) { for (auto& it : sc.items()) normalize_schema_types(it); return; }
  if (!sc.is_object()) return;
  for (auto& kv : sc.members()) {
    const std::string& k = kv.first;
    Json& v = kv.second;
    if (k == "type") {
      if (v.is_string()) v = Json(schema_type_name(v.as_string()));
      else if (v.is_array()) {
        Json out = Json::array();
        for (auto& it : v.items()) {
          Json n = it.is_string() ? Json(schema_type_name(it.as_string())) : it;
          bool seen = false;
          for (auto& o : out.items()) if (o.dump() == n.dump()) seen = true;
          if (!seen) out.push_back(n);
        }
        v = out;
      }
    } else if (k == "properties" || k == "patternProperties" || k == "$defs" || k == "definitions" || k == "dependentSchemas") {
      if (v.is_object()) for (auto& m : v.members()) normalize_schema_types(m.second);
    } else if (k == "anyOf" || k == "oneOf" || k == "allOf" || k == "prefixItems") {
      if (v.is_array()) for (auto& m : v.items()) normalize_schema_types(m);
    } else if (k == "items" || k == "additionalProperties" || k == "not" || k == "if" || k == "then" || k == "else" || k == "contains" ||
               k == "propertyNames" || k == "unevaluatedItems" || k == "unevaluatedProperties") {
      normalize_schema_types(v);
    }
  }
}

static HttpResponse handle_chat(Server& sv, const Json& body, const std::string& session_hdr, Emit* emit) {
  if (!body.is_object()) return error_response(400, "request body must be a JSON object");
  if (std::string e = reject_unsupported(body, true); !e.empty()) return error_response(400, e);
  const Json* ms = body.find("messages");
  if (!ms || !ms->is_array() || ms->size() == 0) return error_response(400, "messages must be a non-empty array");
  std::vector<ChatMessage> msgs;
  Json image_urls = Json::array();
  for (auto& m : ms->items()) {
    ChatMessage cm;
    cm.role = m.get_string("role", "");
    if (cm.role != "system" && cm.role != "user" && cm.role != "assistant" && cm.role != "tool" && cm.role != "developer") return error_response(400, "unknown message role: " + cm.role);
    // with a checkpoint template the role goes through as written (the template decides what it accepts); the built-in
    // ChatML renderer treats "developer" as "system"
    if (cm.role == "developer" && sv.chat_template.empty()) cm.role = "system";
    if (auto c = m.find("content")) {
      if (c->is_string()) cm.content = c->as_string();
      else if (c->is_array()) {
        for (auto& part : c->items()) {
          const std::string type = part.get_string("type", "");
          if (type == "text") {
            // text parts of a tool result are joined with one space, those of other roles run together
            if (cm.role == "tool" && !cm.content.empty()) cm.content += " ";
            cm.content += part.get_string("text", "");
          }
          else if (type == "image_url") {
            if (!sv.backend->supports_images()) return error_response(400, "this model does not accept images");
            const Json* iu = part.find("image_url");
            const std::string url = iu ? iu->get_string("url", "") : "";
            if (url.compare(0, 5, "data:") != 0) return error_response(400, "only base64 data: URLs are accepted for images");
            image_urls.push_back(url);
            cm.content += "<|vision_start|><|image_pad|><|vision_end|>";
          } else return error_response(400, "unsupported content part type: " + type);
        }
      }
    }
    cm.reasoning = m.get_string("reasoning_content", "");
    if (auto tc = m.find("tool_calls")) cm.tool_calls = *tc;
    msgs.push_back(cm);
  }
  bool enable_thinking = true;
  if (auto k = body.find("chat_template_kwargs"); k && k->is_object()) enable_thinking = k->get_bool("enable_thinking", true);
  // reasoning effort: top-level "reasoning_effort" or {"reasoning": {"effort": ...}}; "none" switches thinking off, any
  // other value goes to the template (which knows the values it supports)
  std::string effort = body.get_string("reasoning_effort", "");
  if (auto r = body.find("reasoning"); r && r->is_object() && effort.empty()) effort = r->get_string("effort", "");
  if (effort == "none") { enable_thinking = false; effort.clear(); }
  const bool cont = body.get_bool("continue_final_message", false);
  // A conversation that ends with an assistant message: with continue_final_message the turn is reopened and its
  // text continued; without it the text is handed to the model as a user message (request corpus: assistant_last_converted)
  std::string continue_text;
  if (!sv.chat_template.empty() && !msgs.empty() && msgs.back().role == "assistant") {
    if (cont) { continue_text = msgs.back().content; msgs.pop_back(); }
    else msgs.back().role = "user";
  }
  const Json tools = body.find("tools") && body.at("tools").is_array() && body.get_string("tool_choice", "auto") != "none" ? body.at("tools") : Json::array();
  {
    // tool_choice against the tools, and the token cap against the context (openai.rs:671-706 of the reference)
    const bool has_tools = body.find("tools") && body.at("tools").is_array() && body.at("tools").size() > 0;
    const Json* tc = body.find("tool_choice");
    if (tc && tc->is_string() && tc->as_string() == "required" && !has_tools)
      return error_response(400, "Tools cannot be empty if tool choice is set to required.");
    if (tc && tc->is_object()) {
      std::string name;
      if (auto fn = tc->find("function"); fn && fn->is_object()) name = fn->get_string("name", "");
      if (!has_tools) return error_response(400, "Tools cannot be empty if tool choice is set to a specific tool.");
      bool exists = false;
      for (auto& t : body.at("tools").items())
        if (auto fn = t.find("function"); fn && fn->is_object() && fn->get_string("name", "") == name) exists = true;
      if (!exists) return error_response(400, "Tool '" + name + "' not found in tools list.");
    }
    long long cap = 0;
    if (auto p = body.find("max_completion_tokens"); p && p->is_number() && p->as_int() != 0) cap = p->as_int();
    else if (auto q = body.find("max_tokens"); q && q->is_number()) cap = q->as_int();
    const long long ctx_len = sv.backend->context_length();
    if (cap != 0 && cap > ctx_len)
      return error_response(400, "max_completion_tokens is too large: " + std::to_string(cap) + ".This model supports at most " +
                                     std::to_string(ctx_len) + " completion tokens.");
  }
  std::string prompt;
  if (sv.chat_template.empty()) prompt = render_chatml(msgs, tools, !cont, enable_thinking, cont);
  else {
    // the checkpoint's own template: messages as the template families expect them (tool-call arguments as objects)
    Json jm = Json::array();
    for (auto& m : msgs) {
      Json o = Json::object();
      o.set("role", m.role); o.set("content", m.content);
      if (!m.reasoning.empty()) o.set("reasoning_content", m.reasoning);
      if (m.tool_calls.is_array() && m.tool_calls.size()) {
        Json calls = Json::array();
        for (auto& tc : m.tool_calls.items()) {
          Json call = tc;
          if (const Json* fn = tc.find("function"); fn && fn->is_object()) {
            Json f = *fn;
            if (const Json* a = fn->find("arguments"); a && a->is_string()) {
              try { f.set("arguments", Json::parse(a->as_string())); }
              catch (const std::exception&) { return error_response(400, "Assistant tool call function.arguments must be valid JSON.", "BadRequest"); }
              if (!f.at("arguments").is_object()) return error_response(400, "Assistant tool call function.arguments must be a JSON object.", "BadRequest");
            }
            call.set("function", f);
          }
          calls.push_back(call);
        }
        o.set("tool_calls", calls);
      }
      if (!m.tool_call_id.empty()) o.set("tool_call_id", m.tool_call_id);
      jm.push_back(o);
    }
    Json ctx = Json::object();
    ctx.set("messages", jm);
    std::string forced_tool;
    if (auto tc = body.find("tool_choice"); tc && tc->is_object())
      if (auto fn = tc->find("function"); fn && fn->is_object()) forced_tool = fn->get_string("name", "");
    if (tools.size()) {
      // tools as the reference hands them to its template: the function's fields in the order description, name,
      // parameters (then whatever else the request carried), the parameter schema as written
      Json norm = Json::array();
      for (auto& t : tools.items()) {
        const Json* fn = t.find("function");
        if (!fn || !fn->is_object()) { norm.push_back(t); continue; }
        if (!forced_tool.empty() && fn->get_string("name", "") != forced_tool) continue;   // a named tool_choice lists that tool only
        Json f = Json::object();
        f.set("description", fn->find("description") ? *fn->find("description") : Json());
        f.set("name", fn->find("name") ? *fn->find("name") : Json());
        Json params = fn->find("parameters") ? *fn->find("parameters") : Json();
        normalize_schema_types(params);
        f.set("parameters", params);
        f.set("strict", fn->find("strict") && fn->at("strict").is_bool() ? fn->at("strict") : Json(false));
        const Json* defer = t.find("defer_loading");
        if (defer && !defer->is_null()) f.set("defer_loading", *defer);
        Json o = Json::object();
        o.set("type", t.find("type") ? *t.find("type") : Json("function"));
        o.set("function", f);
        o.set("defer_loading", defer ? *defer : Json());
        norm.push_back(o);
      }
      ctx.set("tools", norm);
    }
    ctx.set("add_generation_prompt", continue_text.empty() ? !cont : true);
    ctx.set("enable_thinking", enable_thinking);
    if (!effort.empty()) ctx.set("reasoning_effort", effort);
    ctx.set("bos_token", sv.bos_token); ctx.set("eos_token", sv.eos_token);
    if (auto k = body.find("chat_template_kwargs"); k && k->is_object()) for (auto& kv : k->members()) ctx.set(kv.first, kv.second);
    try { prompt = render_jinja(sv.chat_template, ctx); }
    catch (const std::exception& e) { return error_response(400, e.what(), "BadRequest"); }
    if (!continue_text.empty()) {
      prompt += continue_text;               // the reopened assistant turn continues where its text stopped
    } else if (cont && !msgs.empty()) {
      // continue_final_message on another role: cut the rendering after the last message's content (the turn stays open)
      const std::string& last = msgs.back().content;
      const size_t at = last.empty() ? std::string::npos : prompt.rfind(last);
      if (at != std::string::npos) prompt.resize(at + last.size());
    }
  }
  Json sampling;
  if (std::string e = build_sampling(sv, body, true, sampling); !e.empty()) return error_response(400, e);
  if (auto rb = body.find("reasoning_budget"); rb && rb->is_number()) sampling.set("reasoning_budget", rb->as_int());
  if (image_urls.size()) sampling.set("images", image_urls);      // one per placeholder, in prompt order
  const std::vector<int> ids = sv.tok.encode(prompt);
  if ((long long)ids.size() >= sv.backend->context_length()) return error_response(400, "the prompt is longer than the model's context length");
  const std::string session = !session_hdr.empty() ? session_hdr : body.get_string("session_id", "");
  // a template that opens the think block itself leaves the generation inside it
  const size_t last_open = prompt.rfind(sv.tags.think_open), last_close = prompt.rfind(sv.tags.think_close);
  const bool in_think = !sv.chat_template.empty() && last_open != std::string::npos &&
                        (last_close == std::string::npos || last_close < last_open);
  return run_generation(sv, body, true, ids, sampling, in_think, session, emit, enable_thinking);
}

static HttpResponse handle_completion(Server& sv, const Json& body, const std::string& session_hdr, Emit* emit) {
  if (!body.is_object()) return error_response(400, "request body must be a JSON object");
  if (std::string e = reject_unsupported(body, false); !e.empty()) return error_response(400, e);
  const Json* p = body.find("prompt");
  std::vector<int> ids;
  if (!p) return error_response(400, "prompt is required");
  if (p->is_string()) ids = sv.tok.encode(p->as_string());
  else if (p->is_array() && p->size() && (*p)[0].is_int()) for (auto& v : p->items()) ids.push_back((int)v.as_int());
  else if (p->is_array() && p->size() == 1 && (*p)[0].is_string()) ids = sv.tok.encode((*p)[0].as_string());
  else return error_response(400, "prompt must be one string or one list of token ids (batched prompts are not supported)");
  Json sampling;
  if (std::string e = build_sampling(sv, body, false, sampling); !e.empty()) return error_response(400, e);
  const std::string session = !session_hdr.empty() ? session_hdr : body.get_string("session_id", "");
  return run_generation(sv, body, false, ids, sampling, false, session, emit);
}

static HttpResponse route(Server& sv, const std::string& method, const std::string& path, const std::string& session_hdr,
                          const std::string& body_text, Emit* emit) {
  if (method == "GET" && (path == "/health" || path == "/health_generate")) { HttpResponse r; r.content_type = "text/plain"; return r; }
  if (method == "GET" && path == "/metrics") {
    HttpResponse r; r.content_type = "text/plain; version=0.0.4";
    std::ostringstream o;
    o << "b200e_requests_total " << sv.n_requests << "\nb200e_prompt_tokens_total " << sv.n_prompt_tokens
      << "\nb200e_completion_tokens_total " << sv.n_completion_tokens << "\nb200e_errors_total " << sv.n_errors << "\n";
    { std::lock_guard<std::mutex> l(sv.extra_mu); o << sv.extra_metrics; }
    r.body = o.str();
    return r;
  }
  auto model_card = [&]() { Json m = Json::object(); m.set("id", sv.model_name); m.set("object", "model"); m.set("created", (long long)std::time(nullptr)); m.set("engine_version", "0.1.0"); m.set("owned_by", "b200-engine"); m.set("root", sv.model_name); m.set("parent", Json()); m.set("max_model_len", sv.backend->context_length()); return m; };   // the reference's card: id, object, created, version, owned_by, root, parent, max_model_len
  if (method == "GET" && path == "/v1/models") { Json o = Json::object(), a = Json::array(); a.push_back(model_card()); o.set("object", "list"); o.set("data", a); HttpResponse r; r.body = o.dump(); return r; }
  if (method == "GET" && path.compare(0, 11, "/v1/models/") == 0) {
    if (path.substr(11) != sv.model_name) return error_response(404, "model not found: " + path.substr(11), "NotFoundError");
    HttpResponse r; r.body = model_card().dump(); return r;
  }
  if (method == "POST" && (path == "/v1/chat/completions" || path == "/v1/completions")) {
    Json body;
    try { body = Json::parse(body_text); } catch (const std::exception& e) { return error_response(400, std::string("invalid JSON: ") + e.what()); }
    return path == "/v1/chat/completions" ? handle_chat(sv, body, session_hdr, emit) : handle_completion(sv, body, session_hdr, emit);
  }
  return error_response(404, "no route for " + method + " " + path, "NotFoundError");
}

// ------------------------------------------------------------------------------------------------ HTTP/1.1 over sockets
static bool send_all(int fd, const std::string& s) {
  size_t off = 0;
  while (off < s.size()) { ssize_t n = ::send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL); if (n <= 0) return false; off += (size_t)n; }
  return true;
}
static const char* status_text(int s) { return s == 200 ? "OK" : s == 400 ? "Bad Request" : s == 404 ? "Not Found" : s == 500 ? "Internal Server Error" : "Error"; }

// Limits of the socket layer: a request head of at most 1 MiB, a body of at most kMaxBody bytes, kIoTimeoutS seconds of
// silence while a request is being read, and at most kMaxConnections connections being served at once.
constexpr size_t kMaxBody = 512ull << 20;
constexpr int kIoTimeoutS = 30;
constexpr int kMaxConnections = 2048;
static std::atomic<int> g_connections{0};

static void send_plain(int fd, int status, const std::string& body) {
  std::ostringstream o;
  o << "HTTP/1.1 " << status << " " << (status == 413 ? "Payload Too Large" : status == 408 ? "Request Timeout" : status == 503 ? "Service Unavailable" : status_text(status))
    << "\r\nContent-Type: application/json\r\nContent-Length: " << body.size() << "\r\nConnection: close\r\n\r\n" << body;
  send_all(fd, o.str());
}

static void serve_connection_inner(Server* sv, int fd) {
  timeval tv{kIoTimeoutS, 0};
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
  std::string buf;
  char tmp[8192];
  size_t hdr_end = std::string::npos;
  while (hdr_end == std::string::npos) {
    ssize_t n = recv(fd, tmp, sizeof tmp, 0);
    if (n <= 0) return;
    const size_t from = buf.size() < 3 ? 0 : buf.size() - 3;
    buf.append(tmp, (size_t)n);
    hdr_end = buf.find("\r\n\r\n", from);
    if (hdr_end == std::string::npos && buf.size() > (1 << 20)) { send_plain(fd, 400, error_response(400, "request head too large").body); return; }
  }
  std::istringstream hs(buf.substr(0, hdr_end));
  std::string method, path, ver, line, session;
  hs >> method >> path >> ver;
  size_t clen = 0;
  bool expect_continue = false, chunked = false;
  std::getline(hs, line);
  while (std::getline(hs, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    const size_t c = line.find(':');
    if (c == std::string::npos) continue;
    std::string k = line.substr(0, c), v = line.substr(c + 1);
    while (!v.empty() && (v[0] == ' ' || v[0] == '\t')) v.erase(0, 1);
    while (!v.empty() && (v.back() == ' ' || v.back() == '\t')) v.pop_back();
    for (auto& ch : k) ch = (char)tolower((unsigned char)ch);
    if (k == "content-length") {
      if (v.empty() || v.size() > 18 || v.find_first_not_of("0123456789") != std::string::npos) { send_plain(fd, 400, error_response(400, "bad Content-Length").body); return; }
      clen = (size_t)std::strtoull(v.c_str(), nullptr, 10);
    }
    if (k == "x-session-id") session = v;
    if (k == "expect") { std::string lv = v; for (auto& ch : lv) ch = (char)tolower((unsigned char)ch); expect_continue = lv == "100-continue"; }
    if (k == "transfer-encoding") { std::string lv = v; for (auto& ch : lv) ch = (char)tolower((unsigned char)ch); chunked = lv.find("chunked") != std::string::npos; }
  }
  if (clen > kMaxBody) { send_plain(fd, 413, error_response(413, "request body too large").body); return; }
  std::string body = buf.substr(hdr_end + 4);
  if (expect_continue && body.size() < clen) send_all(fd, "HTTP/1.1 100 Continue\r\n\r\n");
  if (chunked) {
    // chunked request body: size line (hex, optional extensions), data, CRLF ... until a zero-size chunk
    std::string raw = std::move(body);
    body.clear();
    size_t p = 0;
    auto need = [&](size_t upto) {
      while (raw.size() < upto) { ssize_t n = recv(fd, tmp, sizeof tmp, 0); if (n <= 0) return false; raw.append(tmp, (size_t)n); if (raw.size() > kMaxBody + (1 << 20)) return false; }
      return true;
    };
    for (;;) {
      size_t eol;
      while ((eol = raw.find("\r\n", p)) == std::string::npos) { if (raw.size() - p > 64 || !need(raw.size() + 1)) { send_plain(fd, 400, error_response(400, "bad chunked body").body); return; } }
      const std::string sz = raw.substr(p, eol - p);
      char* endp = nullptr;
      const unsigned long long n = std::strtoull(sz.c_str(), &endp, 16);
      if (endp == sz.c_str() || n > kMaxBody || body.size() + n > kMaxBody) { send_plain(fd, endp == sz.c_str() ? 400 : 413, error_response(400, "bad chunked body").body); return; }
      p = eol + 2;
      if (n == 0) break;
      if (!need(p + n + 2)) { send_plain(fd, 400, error_response(400, "truncated chunked body").body); return; }
      body.append(raw, p, (size_t)n);
      p += n + 2;
    }
  } else {
    body.reserve(std::min(clen, (size_t)(64u << 20)));
    while (body.size() < clen) { ssize_t n = recv(fd, tmp, sizeof tmp, 0); if (n <= 0) break; body.append(tmp, (size_t)n); }
    if (body.size() < clen) { send_plain(fd, 408, error_response(408, "request body incomplete").body); return; }
    if (body.size() > clen) body.resize(clen);
  }
  const size_t q = path.find('?');
  if (q != std::string::npos) path.resize(q);
  bool headers_sent = false, alive = true;
  Emit em;
  em.write = [&](const std::string& ev) {
    if (!headers_sent) { alive = send_all(fd, "HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\nConnection: close\r\n\r\n"); headers_sent = true; }
    if (alive) alive = send_all(fd, ev);
  };
  em.alive = [&]() {
    if (!alive) return false;
    char c;
    const ssize_t n = recv(fd, &c, 1, MSG_PEEK | MSG_DONTWAIT);
    if (n == 0) alive = false;      // orderly shutdown by the client
    return alive;
  };
  HttpResponse r;
  try {
    r = route(*sv, method, path, session, body, &em);
  } catch (const std::exception& e) {                 // a handler's bug must not take the process down
    r = error_response(500, std::string("internal error: ") + e.what(), "InternalServerError");
  } catch (...) {
    r = error_response(500, "internal error", "InternalServerError");
  }
  if (!(r.sse && headers_sent)) {
    std::ostringstream o;
    o << "HTTP/1.1 " << r.status << " " << status_text(r.status) << "\r\nContent-Type: " << r.content_type << "\r\nContent-Length: " << r.body.size() << "\r\nConnection: close\r\n\r\n";
    send_all(fd, o.str() + r.body);
  }
}

static void serve_connection(Server* sv, int fd) {
  serve_connection_inner(sv, fd);
  shutdown(fd, SHUT_RDWR);
  close(fd);
  --g_connections;
  --sv->live_connections;                    // last use of sv by this thread
}

// Connection threads are detached; the object they serve must outlive them.  Waits (bounded) until none is left.
static void drain_connections(Server* sv, int seconds) {
  for (int i = 0; i < seconds * 100 && sv->live_connections.load() > 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(10));
}

}  // namespace b2

using namespace b2;

static char* dup_cstr(const std::string& s) { char* p = (char*)malloc(s.size() + 1); memcpy(p, s.c_str(), s.size() + 1); return p; }

// config: {"tokenizer_json": path, "model_name", "generation_config": {...}, "eos_token_ids": [..], "max_tokens_default"}
B2H_API void* b2h_server_new(const char* config_json, char* err, int err_cap) {
  try {
    Json c = Json::parse(config_json);
    auto sv = new Server();
    if (auto p = c.find("tokenizer_json"); p && p->is_string()) {
      std::ifstream f(p->as_string());
      if (!f) throw std::runtime_error("cannot read " + p->as_string());
      std::stringstream ss; ss << f.rdbuf();
      sv->tok = Tokenizer::from_json(ss.str());
      sv->has_tok = true;
    }
    sv->model_name = c.get_string("model_name", "b200-engine");
    if (auto g = c.find("generation_config"); g && g->is_object()) sv->gen_defaults = *g;
    if (auto e = c.find("eos_token_ids"); e && e->is_array()) for (auto& v : e->items()) sv->eos_ids.push_back((int)v.as_int());
    if (sv->eos_ids.empty()) {                 // generation_config.json names the end-of-sequence ids (one id or a list)
      if (auto e = sv->gen_defaults.find("eos_token_id")) {
        if (e->is_int()) sv->eos_ids.push_back((int)e->as_int());
        else if (e->is_array()) for (auto& v : e->items()) if (v.is_int()) sv->eos_ids.push_back((int)v.as_int());
      }
    }
    sv->max_tokens_default = c.get_int("max_tokens_default", 32768);
    sv->chat_template = c.get_string("chat_template", "");
    sv->bos_token = c.get_string("bos_token", "");
    sv->eos_token = c.get_string("eos_token", "");
    if (sv->chat_template.find("<|think|>") != std::string::npos) { sv->tags.think_open = "<|think|>"; sv->tags.think_close = "<|/think|>"; }
    if (sv->chat_template.find("<|call|>") != std::string::npos) { sv->tags.call_open = "<|call|>"; sv->tags.call_close = "<|/call|>"; }
    if (sv->has_tok) sv->think_close_ids = sv->tok.encode(sv->tags.think_close);
    sv->backend = std::make_shared<MockBackend>();
    return sv;
  } catch (const std::exception& e) { if (err) snprintf(err, err_cap, "%s", e.what()); return nullptr; }
}
B2H_API void b2h_server_stop(void* sp);
B2H_API void b2h_server_free(void* s) {
  auto sv = static_cast<Server*>(s);
  if (sv->listen_fd.load() >= 0 || sv->accept_thread.joinable()) b2h_server_stop(s);
  drain_connections(sv, 30);
  if (sv->live_connections.load() > 0) return;            // a connection is stuck past every time-out: leak rather than free under it
  delete sv;
}
B2H_API void b2h_server_use_mock(void* s, const int* script, int n, int step, int supports_images) {
  auto m = std::make_shared<MockBackend>();
  m->script.assign(script, script + n); m->step = std::max(1, step); m->images = supports_images != 0;
  static_cast<Server*>(s)->backend = m;
}
// JSON list of the calls the mock backend received: [{"prompt": [...], "sampling": {...}, "session_id": "..."}]
B2H_API char* b2h_server_mock_calls(void* s) {
  auto m = std::dynamic_pointer_cast<MockBackend>(static_cast<Server*>(s)->backend);
  Json a = Json::array();
  if (m) { std::lock_guard<std::mutex> l(m->mu); for (auto& c : m->calls) { Json o = Json::object(), p = Json::array(); for (int t : c.prompt) p.push_back(t); o.set("prompt", p); o.set("sampling", c.sampling); o.set("session_id", c.session_id); a.push_back(o); } }
  return dup_cstr(a.dump());
}
// Replaces the engine-side part of /metrics (Prometheus text lines, newline terminated).
B2H_API void b2h_server_set_metrics(void* s, const char* text) {
  auto sv = static_cast<Server*>(s);
  std::lock_guard<std::mutex> l(sv->extra_mu);
  sv->extra_metrics = text ? text : "";
}
B2H_API int b2h_server_set_images(void* s, int on) {
  auto b = std::dynamic_pointer_cast<CallbackBackend>(static_cast<Server*>(s)->backend);
  if (!b) return -1;
  b->images = on != 0;
  return 0;
}
B2H_API void b2h_server_use_callback(void* s, GenerateFn fn, void* user, int context_length) {
  auto b = std::make_shared<CallbackBackend>();
  b->fn = fn; b->user = user; b->ctx = context_length;
  static_cast<Server*>(s)->backend = b;
}
// Engine side of the callback backend: push a step's tokens / finish / fail; ask whether the client is gone.
B2H_API int b2h_stream_push(void* s, long long req_id, const int* ids, int n, int finished, const char* error) {
  auto b = std::dynamic_pointer_cast<CallbackBackend>(static_cast<Server*>(s)->backend);
  if (!b) return -1;
  auto ts = b->find(req_id);
  if (!ts) return -1;
  ts->push(ids, n, finished != 0, error);
  return ts->is_cancelled() ? 1 : 0;
}
B2H_API int b2h_stream_cancelled(void* s, long long req_id) {
  auto b = std::dynamic_pointer_cast<CallbackBackend>(static_cast<Server*>(s)->backend);
  if (!b) return 1;
  auto ts = b->find(req_id);
  return !ts || ts->is_cancelled() ? 1 : 0;
}
// In-process request (tests, embedding): returns the full body; *status receives the HTTP status.
B2H_API char* b2h_server_handle(void* s, const char* method, const char* path, const char* session_id, const char* body, int* status) {
  HttpResponse r = route(*static_cast<Server*>(s), method, path, session_id ? session_id : "", body ? body : "", nullptr);
  if (status) *status = r.status;
  return dup_cstr(r.body);
}
// Starts listening (port 0 = any free port); returns the bound port or -1.
B2H_API int b2h_server_start(void* sp, const char* host, int port) {
  auto sv = static_cast<Server*>(sp);
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{};
  a.sin_family = AF_INET; a.sin_port = htons((uint16_t)port);
  if (inet_pton(AF_INET, host && *host ? host : "127.0.0.1", &a.sin_addr) != 1) { close(fd); return -1; }
  if (bind(fd, (sockaddr*)&a, sizeof a) != 0 || listen(fd, 128) != 0) { close(fd); return -1; }
  socklen_t len = sizeof a;
  getsockname(fd, (sockaddr*)&a, &len);
  sv->listen_fd = fd;
  sv->stopping = false;
  sv->accept_thread = std::thread([sv]() {
    while (!sv->stopping) {
      const int lfd = sv->listen_fd.load();
      if (lfd < 0) break;
      int c = accept(lfd, nullptr, nullptr);
      if (c < 0) { if (sv->stopping) break; continue; }
      int one = 1;
      setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
      if (++g_connections > kMaxConnections) {            // shed load instead of piling up threads
        send_plain(c, 503, error_response(503, "too many connections").body);
        close(c);
        --g_connections;
        continue;
      }
      ++sv->live_connections;
      try {
        std::thread(serve_connection, sv, c).detach();
      } catch (const std::system_error&) { close(c); --g_connections; --sv->live_connections; }
    }
  });
  return ntohs(a.sin_port);
}
B2H_API void b2h_server_stop(void* sp) {
  auto sv = static_cast<Server*>(sp);
  sv->stopping = true;
  const int lfd = sv->listen_fd.exchange(-1);
  if (lfd >= 0) { shutdown(lfd, SHUT_RDWR); close(lfd); }
  if (sv->accept_thread.joinable()) sv->accept_thread.join();
  drain_connections(sv, 5);                  // requests in flight finish (or their clients time out) before the caller moves on
}

// ---- text layer exports (tests, Python-side engine glue) ----
B2H_API void* b2h_tok_new(const char* tokenizer_json_text, char* err, int cap) {
  try { return new Tokenizer(Tokenizer::from_json(tokenizer_json_text)); } catch (const std::exception& e) { if (err) snprintf(err, cap, "%s", e.what()); return nullptr; }
}
B2H_API void b2h_tok_free(void* t) { delete static_cast<Tokenizer*>(t); }
B2H_API int b2h_tok_encode(void* t, const char* text, int* out, int cap) {
  auto ids = static_cast<Tokenizer*>(t)->encode(text);
  for (int i = 0; i < (int)ids.size() && i < cap; ++i) out[i] = ids[i];
  return (int)ids.size();
}
B2H_API char* b2h_tok_decode(void* t, const int* ids, int n, int skip_special) {
  return dup_cstr(static_cast<Tokenizer*>(t)->decode(std::vector<int>(ids, ids + n), skip_special != 0));
}
B2H_API void* b2h_detok_new(void* t, int skip_special) { return new Detokenizer(static_cast<Tokenizer*>(t), skip_special != 0); }
B2H_API void b2h_detok_free(void* d) { delete static_cast<Detokenizer*>(d); }
B2H_API char* b2h_detok_push(void* d, const int* ids, int n) { return dup_cstr(static_cast<Detokenizer*>(d)->push(std::vector<int>(ids, ids + n))); }
B2H_API char* b2h_detok_finish(void* d) { return dup_cstr(static_cast<Detokenizer*>(d)->finish()); }
// messages: JSON array of {role, content, reasoning_content?, tool_calls?}
B2H_API char* b2h_render_chat(const char* messages_json, const char* tools_json, int add_generation_prompt, int enable_thinking, int continue_final) {
  try {
    Json ms = Json::parse(messages_json), tools = tools_json && *tools_json ? Json::parse(tools_json) : Json::array();
    std::vector<ChatMessage> msgs;
    for (auto& m : ms.items()) { ChatMessage c; c.role = m.get_string("role", ""); c.content = m.get_string("content", ""); c.reasoning = m.get_string("reasoning_content", ""); if (auto t = m.find("tool_calls")) c.tool_calls = *t; msgs.push_back(c); }
    return dup_cstr(render_chatml(msgs, tools, add_generation_prompt != 0, enable_thinking != 0, continue_final != 0));
  } catch (const std::exception& e) { return dup_cstr(std::string("ERROR: ") + e.what()); }
}
// Parses text in chunks of `chunk` bytes (0 = at once); returns {"content", "reasoning", "tool_calls": [{name, arguments}]}.
// Renders a Jinja chat template with a JSON object of variables.  On failure returns null and writes the message to err.
B2H_API char* b2h_render_template(const char* source, const char* context_json, char* err, int err_cap) {
  try {
    return dup_cstr(render_jinja(source, Json::parse(context_json)));
  } catch (const std::exception& e) {
    if (err && err_cap > 0) { std::strncpy(err, e.what(), (size_t)err_cap - 1); err[err_cap - 1] = 0; }
    return nullptr;
  }
}
static char* parse_output_with(const char* text, const char* tools_json, int starts_in_reasoning, int chunk,
                               const std::string& think_open, const std::string& think_close,
                               const std::string& call_open, const std::string& call_close);
B2H_API char* b2h_parse_output(const char* text, const char* tools_json, int starts_in_reasoning, int chunk) {
  return parse_output_with(text, tools_json, starts_in_reasoning, chunk, "<think>", "</think>", "<tool_call>", "</tool_call>");
}
// The same with the tags of another template family (the reference model writes <|think|>, <|/think|>, <|call|>, <|/call|>).
B2H_API char* b2h_parse_output_tags(const char* text, const char* tools_json, int starts_in_reasoning, int chunk,
                                    const char* think_open, const char* think_close, const char* call_open, const char* call_close) {
  return parse_output_with(text, tools_json, starts_in_reasoning, chunk, think_open, think_close, call_open, call_close);
}
static char* parse_output_with(const char* text, const char* tools_json, int starts_in_reasoning, int chunk,
                               const std::string& think_open, const std::string& think_close,
                               const std::string& call_open, const std::string& call_close) {
  Json tools = tools_json && *tools_json ? Json::parse(tools_json) : Json::array();
  const bool with_calls = !tools.is_null();      // "null": the request carries no tools (or tool_choice none): calls stay text
  std::string t = text, content, reasoning;
  std::vector<ToolCall> calls;
  ReasoningParser rp(starts_in_reasoning != 0, true, think_open, think_close);
  ToolStreamParser tp(with_calls ? tools : Json::array(), call_open, call_close);
  if (think_open != "<think>") rp.keep_newlines_after_close(true);
  if (call_open != "<tool_call>" && with_calls) {          // the other template family: its parsers' conventions
    rp.set_interrupt(call_open);
    tp.content_before_calls_only(true);
  }
  auto feed = [&](const std::string& piece, bool last) {
    auto ro = rp.push(piece);
    if (last) { auto f = rp.finish(); ro.content += f.content; ro.reasoning += f.reasoning; }
    reasoning += ro.reasoning;
    if (!with_calls) { content += ro.content; return; }
    auto tr = tp.push(ro.content);
    if (last) { auto f = tp.finish(); tr.content += f.content; for (auto& c : f.calls) tr.calls.push_back(c); }
    content += tr.content;
    for (auto& c : tr.calls) calls.push_back(c);
  };
  // A complete (non-streamed) output that was not forced into reasoning but carries the opening tag somewhere is read
  // as reasoning up to its first closing tag, the opening tag's text included (parser corpus: think_start_mid).
  const size_t close_at = t.find(think_close);
  if (chunk <= 0 && !starts_in_reasoning && !think_open.empty() && close_at != std::string::npos &&
      t.find(think_open) != std::string::npos && t.compare(0, think_open.size(), think_open) != 0) {
    reasoning = t.substr(0, close_at);
    ReasoningParser plain(false, true, "\x01no-open\x01", "\x01no-close\x01");
    rp = plain;
    feed(t.substr(close_at + think_close.size()), true);
  } else if (chunk <= 0) feed(t, true);
  else { for (size_t i = 0; i < t.size(); i += (size_t)chunk) feed(t.substr(i, (size_t)chunk), false); feed("", true); }
  Json o = Json::object(), a = Json::array();
  for (auto& c : calls) { Json j = Json::object(); j.set("name", c.name); j.set("arguments", c.arguments_json); a.push_back(j); }
  o.set("content", content); o.set("reasoning", reasoning); o.set("tool_calls", a);
  return dup_cstr(o.dump());
}
