// Text layer of the server: byte-level BPE tokenizer (Hugging Face tokenizer.json), incremental detokenizer,
// chat template, reasoning splitter and tool-call parsers.  See text.cpp for the behaviour each class keeps.
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/json.hpp"

namespace b2 {

class Tokenizer {
 public:
  // Loads vocab, merges and added tokens from tokenizer.json text.  Throws std::runtime_error on malformed input.
  static Tokenizer from_json(const std::string& text);
  std::vector<int> encode(const std::string& text) const;                  // added/special tokens are matched first
  std::string decode(const std::vector<int>& ids, bool skip_special) const;
  std::string token_bytes(int id) const;                                   // raw bytes of one token ("" if unknown)
  bool is_special(int id) const { return special_.count(id) != 0; }
  int token_to_id(const std::string& s) const;                             // added tokens and plain vocab entries
  int size() const { return (int)id_to_tok_.size(); }

 private:
  std::vector<std::string> pretokenize(const std::string& text) const;
  void bpe(const std::string& piece, std::vector<int>& out) const;
  std::unordered_map<std::string, int> vocab_;              // byte-level string -> id
  std::vector<std::string> id_to_tok_;                      // id -> byte-level string (or added-token text)
  std::unordered_map<std::string, int> merge_rank_;         // "a b" -> rank
  std::vector<std::pair<std::string, int>> added_;          // added tokens, longest first
  bool added_first_[256] = {};                              // bytes an added token starts with
  std::unordered_map<int, bool> special_;
  std::unordered_map<int, bool> is_added_;
  // ids of pre-tokens seen before (words repeat: most of a prompt is served from here); shared by the threads that
  // encode through this tokenizer, copies of the tokenizer share it too
  struct WordCache { std::shared_mutex mu; std::unordered_map<std::string, std::vector<int>> ids; };
  std::shared_ptr<WordCache> cache_ = std::make_shared<WordCache>();
};

// Streams text out of a growing id list without ever emitting half a UTF-8 sequence.
class Detokenizer {
 public:
  Detokenizer(const Tokenizer* tk, bool skip_special) : tk_(tk), skip_special_(skip_special) {}
  std::string push(const std::vector<int>& ids);   // returns the text that became final
  std::string finish();                            // flushes held-back bytes (invalid tails become U+FFFD)
 private:
  const Tokenizer* tk_;
  bool skip_special_;
  std::string pending_;
};

struct ChatMessage { std::string role, content, reasoning; Json tool_calls; std::string tool_call_id; };

// ChatML rendering (the template family of the dense GQA checkpoints): system/user/assistant/tool turns, a tools
// preamble, generation prompt, optional disabled thinking (empty think block) and continue_final_message.
std::string render_chatml(const std::vector<ChatMessage>& msgs, const Json& tools, bool add_generation_prompt,
                          bool enable_thinking, bool continue_final);

// Renders a Jinja chat template (the subset in jinja.cpp) with the variables of `context`; throws std::runtime_error.
std::string render_jinja(const std::string& source, const Json& context);

// Splits generated text into reasoning and content around <think> ... </think>.
class ReasoningParser {
 public:
  ReasoningParser(bool starts_in_reasoning, bool stream_reasoning, std::string open = "<think>", std::string close = "</think>")
      : in_(starts_in_reasoning), stream_(stream_reasoning), open_(std::move(open)), close_(std::move(close)) {}
  struct Out { std::string content, reasoning; };
  Out parse_all(const std::string& text) const;
  Out push(const std::string& delta);
  Out finish();
  // A tag that ends an unclosed thinking block when it shows up inside it (the tool-call opener): the model went
  // straight from thinking to a call.  Empty = off.
  void set_interrupt(std::string tag) { interrupt_ = std::move(tag); }
  // Newlines right after the closing tag: dropped by default (the ChatML family writes "</think>\n\n" before the
  // answer); the reference model's parsers hand them on as content.
  void keep_newlines_after_close(bool on) { keep_nl_ = on; }
 private:
  bool in_, stream_;
  std::string open_, close_, interrupt_, buf_, held_reasoning_;
  bool stripped_open_ = false, strip_nl_ = false, keep_nl_ = false;
};

struct ToolCall { std::string name, arguments_json; };

// Tool calls in either wire format: <tool_call>{"name": .., "arguments": {..}}</tool_call> (JSON body) or
// <function=NAME><parameter=KEY>VALUE</parameter>...</function> (typed by the tool's JSON schema).
struct ToolParse {
  std::string content;
  std::vector<ToolCall> calls;
  bool unfinished = false;      // the text ended inside a call: that call is neither reported nor content
};
ToolParse parse_tool_calls(const std::string& text, const Json& tools);
// The same with the call wrapper of another template family (e.g. "<|call|>" ... "<|/call|>").
ToolParse parse_tool_calls(const std::string& text, const Json& tools, const std::string& call_open, const std::string& call_close);

class ToolStreamParser {
 public:
  explicit ToolStreamParser(Json tools, std::string call_open = "<tool_call>", std::string call_close = "</tool_call>")
      : tools_(std::move(tools)), call_open_(std::move(call_open)), call_close_(std::move(call_close)) {}
  // Feeds generated text; returns content that is certainly not part of a call, and calls completed so far.
  ToolParse push(const std::string& delta);
  ToolParse finish();
  // Content is what precedes the first call only: text after a call and an unfinished call at the end are dropped
  // (the reference's tool-call detector reports `normal_text` that way).
  void content_before_calls_only(bool on) { content_before_calls_only_ = on; }
 private:
  Json tools_;
  std::string call_open_, call_close_;
  std::string buf_, tail_;
  bool content_before_calls_only_ = false, saw_call_ = false;
};

// Streaming view of tool calls in the <function=NAME><parameter=KEY>VALUE</parameter>...</function> format inside a call
// wrapper: instead of whole calls it reports what a streaming client gets: content, the start of a call (its name), and
// pieces of the call's arguments object as its parameters complete ("{", "\"key\": value", ", \"key\": value", "}").
// Behaviour follows the reference's streaming detector (crates/agens-server/src/toolcall.rs, ToolCallStreamParser): a
// value is reported when its parameter ends (closing tag, the next parameter or the end of the function), the closing
// brace when </function> arrives, text between and after calls is content, a partial wrapper tag at the end of the
// output is dropped.
struct ToolDelta {
  enum Kind { Content, Start, Args } kind;
  int index;            // call index (Start / Args)
  std::string text;     // content, function name, or a piece of the arguments JSON
};
class ToolDeltaParser {
 public:
  ToolDeltaParser(Json tools, std::string call_open, std::string call_close)
      : tools_(std::move(tools)), open_(std::move(call_open)), close_(std::move(call_close)) {}
  std::vector<ToolDelta> push(const std::string& delta);
  int calls() const { return n_calls_; }
 private:
  enum St { Outside, WantFunction, InBody, InValue, AfterFunction };
  Json tools_;
  std::string open_, close_, buf_, key_;
  const Json* schema_ = nullptr;
  St st_ = Outside;
  int n_calls_ = 0, n_params_ = 0;
  bool opened_ = false;
};

}  // namespace b2
