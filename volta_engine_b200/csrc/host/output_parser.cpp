// Incremental parser of generated text into reasoning, answer text and tool calls, independent of how the
// text is chunked. Handles the tag syntaxes of the supported families:
//   reasoning   <think> ... </think>
//   tool calls  <tool_call>{"name": .., "arguments": {..}}</tool_call>                    (Qwen / Hermes JSON)
//               <tool_call>name\n<arg_key>k</arg_key>\n<arg_value>v</arg_value>...</tool_call>   (GLM)
//               <｜tool▁calls▁begin｜> ... <｜tool▁call▁begin｜>name<｜tool▁sep｜>{json}<｜tool▁call▁end｜>   (DeepSeek)
// Text that could be the beginning of a tag is held back until it is disambiguated.
// Counterpart of src/server/output_parser.cpp in the reference.
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "json.h"

namespace vh {

struct Event {
  int kind;            // 0 text, 1 reasoning, 2 tool call (payload = JSON {"name":..,"arguments":"<json string>"})
  std::string payload;
};

class OutputParser {
 public:
  OutputParser(int family, bool in_reasoning) : family_(family), state_(in_reasoning ? Reasoning : Text) {
    if (family_ == 2) {
      open_call_ = "<\xEF\xBD\x9Ctool\xE2\x96\x81" "call\xE2\x96\x81" "begin\xEF\xBD\x9C>";
      close_call_ = "<\xEF\xBD\x9Ctool\xE2\x96\x81" "call\xE2\x96\x81" "end\xEF\xBD\x9C>";
      noise_ = {"<\xEF\xBD\x9Ctool\xE2\x96\x81" "calls\xE2\x96\x81" "begin\xEF\xBD\x9C>",
                "<\xEF\xBD\x9Ctool\xE2\x96\x81" "calls\xE2\x96\x81" "end\xEF\xBD\x9C>"};
    } else {
      open_call_ = "<tool_call>";
      close_call_ = "</tool_call>";
    }
  }

  void feed(const std::string& chunk, std::vector<Event>& out) {
    buf_ += chunk;
    process(out, false);
  }
  void finish(std::vector<Event>& out) { process(out, true); }
  bool in_reasoning() const { return state_ == Reasoning; }

 private:
  enum State { Text, Reasoning, Call } state_;
  int family_;
  std::string buf_, open_call_, close_call_;
  std::vector<std::string> noise_;
  bool skip_nl_ = false;

  // Length of the longest suffix of s that is a proper prefix of tag.
  static size_t partial_suffix(const std::string& s, const std::string& tag) {
    size_t best = 0;
    for (size_t k = std::min(tag.size() - 1, s.size()); k > 0; --k)
      if (s.compare(s.size() - k, k, tag, 0, k) == 0) { best = k; break; }
    return best;
  }
  void emit(std::vector<Event>& out, int kind, const std::string& s) {
    if (s.empty()) return;
    if (!out.empty() && out.back().kind == kind && kind != 2) out.back().payload += s;
    else out.push_back({kind, s});
  }

  static std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && isspace((unsigned char)s[a])) ++a;
    while (b > a && isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
  }

  void emit_call(std::vector<Event>& out, const std::string& body_raw) {
    std::string body = trim(body_raw), name, args = "{}";
    if (family_ == 2) {   // name <sep> json   (optionally "function<sep>name\n```json\n{..}\n```")
      const std::string sep = "<\xEF\xBD\x9Ctool\xE2\x96\x81sep\xEF\xBD\x9C>";
      size_t p = body.find(sep);
      if (p != std::string::npos) {
        name = trim(body.substr(0, p));
        std::string rest = trim(body.substr(p + sep.size()));
        if (name == "function") {
          size_t nl = rest.find('\n');
          name = trim(rest.substr(0, nl));
          rest = nl == std::string::npos ? "" : rest.substr(nl + 1);
        }
        size_t a = rest.find('{'), b = rest.rfind('}');
        if (a != std::string::npos && b != std::string::npos && b > a) args = rest.substr(a, b - a + 1);
      } else {
        name = body;
      }
    } else if (!body.empty() && body[0] == '{') {   // JSON object with name + arguments
      try {
        Json j = json_parse(body);
        name = j.get_string("name");
        const Json* a = j.find("arguments");
        if (!a) a = j.find("parameters");
        if (a) {
          if (a->is_string()) args = a->s;
          else { args.clear(); json_dump(*a, args); }
        }
      } catch (...) {
        emit(out, 0, open_call_ + body_raw + close_call_);   // not parseable: give the text back
        return;
      }
    } else {   // GLM key/value form
      size_t nl = body.find('\n');
      size_t ak = body.find("<arg_key>");
      size_t name_end = std::min(nl, ak);
      name = trim(body.substr(0, name_end));
      Json obj = Json::object();
      size_t p = 0;
      while ((p = body.find("<arg_key>", p)) != std::string::npos) {
        size_t e = body.find("</arg_key>", p);
        if (e == std::string::npos) break;
        std::string k = trim(body.substr(p + 9, e - p - 9));
        size_t v0 = body.find("<arg_value>", e), v1 = body.find("</arg_value>", e);
        if (v0 == std::string::npos || v1 == std::string::npos) break;
        std::string v = body.substr(v0 + 11, v1 - v0 - 11);
        Json val;
        try { val = json_parse(trim(v)); } catch (...) { val = Json::string(v); }
        obj.set(k, val);
        p = v1 + 12;
      }
      args.clear();
      json_dump(obj, args);
    }
    Json ev = Json::object();
    ev.set("name", Json::string(name));
    ev.set("arguments", Json::string(args));
    std::string s;
    json_dump(ev, s);
    out.push_back({2, s});
  }

  void process(std::vector<Event>& out, bool final) {
    static const std::string think_open = "<think>", think_close = "</think>";
    for (;;) {
      if (state_ == Text) {
        if (skip_nl_) {   // newlines right after a closing tag are dropped, however the text is chunked
          size_t k = 0;
          while (k < buf_.size() && buf_[k] == '\n') ++k;
          buf_.erase(0, k);
          if (buf_.empty()) return;
          skip_nl_ = false;
        }
        // earliest of: <think>, tool-call opener, noise markers
        size_t pt = buf_.find(think_open), pc = buf_.find(open_call_), pn = std::string::npos, nlen = 0;
        for (auto& nz : noise_) { size_t p = buf_.find(nz); if (p < pn) { pn = p; nlen = nz.size(); } }
        size_t first = std::min(pt, std::min(pc, pn));
        if (first == std::string::npos) {
          size_t hold = 0;
          if (!final) {
            hold = std::max(partial_suffix(buf_, think_open), partial_suffix(buf_, open_call_));
            for (auto& nz : noise_) hold = std::max(hold, partial_suffix(buf_, nz));
          }
          emit(out, 0, buf_.substr(0, buf_.size() - hold));
          buf_.erase(0, buf_.size() - hold);
          return;
        }
        emit(out, 0, buf_.substr(0, first));
        if (first == pt) { buf_.erase(0, first + think_open.size()); state_ = Reasoning; }
        else if (first == pc) { buf_.erase(0, first + open_call_.size()); state_ = Call; }
        else buf_.erase(0, first + nlen);
      } else if (state_ == Reasoning) {
        size_t p = buf_.find(think_close);
        if (p == std::string::npos) {
          size_t hold = final ? 0 : partial_suffix(buf_, think_close);
          emit(out, 1, buf_.substr(0, buf_.size() - hold));
          buf_.erase(0, buf_.size() - hold);
          return;
        }
        emit(out, 1, buf_.substr(0, p));
        buf_.erase(0, p + think_close.size());
        skip_nl_ = true;   // swallow the blank lines that separate reasoning from the answer
        state_ = Text;
      } else {   // Call
        size_t p = buf_.find(close_call_);
        if (p == std::string::npos) {
          if (final) { emit_call(out, buf_); buf_.clear(); state_ = Text; }
          return;
        }
        emit_call(out, buf_.substr(0, p));
        buf_.erase(0, p + close_call_.size());
        skip_nl_ = true;
        state_ = Text;
      }
    }
  }
};

}  // namespace vh

using namespace vh;

extern "C" {

// family: 0 = Qwen / Hermes JSON tool calls, 1 = GLM key/value, 2 = DeepSeek markers.
void* vh_parser_new(int family, int in_reasoning) { return new OutputParser(family, in_reasoning != 0); }
void vh_parser_free(void* p) { delete (OutputParser*)p; }

static char* events_to_c(const std::vector<Event>& ev) {
  Json arr = Json::array();
  for (auto& e : ev) {
    Json o = Json::object();
    o.set("kind", Json::integer(e.kind));
    o.set("payload", Json::string(e.payload));
    arr.arr.push_back(o);
  }
  std::string s;
  json_dump(arr, s);
  char* out = (char*)malloc(s.size() + 1);
  memcpy(out, s.c_str(), s.size() + 1);
  return out;
}

// Returns a malloc'ed JSON array of {"kind", "payload"} events (free with vh_free).
char* vh_parser_feed(void* p, const char* chunk, int len) {
  std::vector<Event> ev;
  ((OutputParser*)p)->feed(std::string(chunk, (size_t)len), ev);
  return events_to_c(ev);
}
char* vh_parser_finish(void* p) {
  std::vector<Event> ev;
  ((OutputParser*)p)->finish(ev);
  return events_to_c(ev);
}
int vh_parser_in_reasoning(void* p) { return ((OutputParser*)p)->in_reasoning() ? 1 : 0; }

}  // extern "C"
