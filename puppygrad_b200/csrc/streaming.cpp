// Text-side helpers of the generation API that need no tokenizer of their own: the incremental text
// streamer over a caller-supplied token decoder (src/models/streaming.rs:1-78) and the rate methods of
// GenerationStats (src/models/generation.rs:129-180). Host code only.
#include <cstring>
#include <string>
#include <vector>

#include "common.h"

using namespace pg;

struct pg_text_streamer {
  std::string decoded;  // IncrementalTextStreamer::decoded
};

namespace {

// is_incremental_decode_safe, streaming.rs:76-78: not empty and without U+FFFD (EF BF BD in UTF-8)
bool decode_safe(const std::string& t) { return !t.empty() && t.find("\xEF\xBF\xBD") == std::string::npos; }

// TokenDecoder::decode_tokens through the callback: the callback reports the length it needs, so a second call
// with a larger buffer follows when the first did not fit.
int call_decoder(pg_decode_tokens_fn decoder, void* user, const uint64_t* ids, size_t n, std::string* out) {
  std::vector<char> buf(256);
  for (int attempt = 0; attempt < 2; ++attempt) {
    size_t len = 0;
    if (decoder(ids, n, buf.data(), buf.size(), &len, user) != 0)
      return set_error(PG_INVALID_INPUT, "token decoder failed");
    if (len <= buf.size()) {
      out->assign(buf.data(), len);
      return PG_OK;
    }
    buf.resize(len);
  }
  return set_error(PG_INVALID_INPUT, "token decoder reported inconsistent lengths");
}

double rate(uint64_t tokens, double seconds) { return seconds == 0.0 ? 0.0 : (double)tokens / seconds; }  // generation.rs:175-181

}  // namespace

extern "C" {

int pg_text_streamer_new(const char* decoded, size_t len, pg_text_streamer** out) {
  if (!out || (!decoded && len)) return set_error(PG_INVALID_INPUT, "null argument");
  *out = new pg_text_streamer{std::string(decoded ? decoded : "", len)};
  return PG_OK;
}

void pg_text_streamer_free(pg_text_streamer* s) { delete s; }

int pg_text_streamer_decoded(const pg_text_streamer* s, const char** text, size_t* len) {
  if (!s || !text || !len) return set_error(PG_INVALID_INPUT, "null argument");
  *text = s->decoded.data();
  *len = s->decoded.size();
  return PG_OK;
}

int pg_text_streamer_stream_token(pg_text_streamer* s, pg_decode_tokens_fn decoder, void* decoder_user,
                                  const uint64_t* output_ids, size_t n_ids, uint64_t token_id, pg_text_callback on_text,
                                  void* text_user) {
  if (!s || !decoder || !on_text || (!output_ids && n_ids)) return set_error(PG_INVALID_INPUT, "null argument");
  auto emit = [&](const std::string& t) -> int {
    if (on_text(t.data(), t.size(), text_user) != 0) return set_error(PG_INVALID_INPUT, "text callback aborted generation");
    return PG_OK;
  };
  std::string token_text;
  if (int r = call_decoder(decoder, decoder_user, &token_id, 1, &token_text)) return r;  // decode_token
  if (decode_safe(token_text)) {
    if (int r = emit(token_text)) return r;
    s->decoded += token_text;
    return PG_OK;
  }
  // the token alone does not decode to text (a partial UTF-8 sequence, an empty piece): decode everything and
  // emit what is new
  std::string next;
  if (int r = call_decoder(decoder, decoder_user, output_ids, n_ids, &next)) return r;
  if (next.compare(0, s->decoded.size(), s->decoded) == 0 && next.size() >= s->decoded.size()) {
    if (int r = emit(next.substr(s->decoded.size()))) return r;
  } else if (int r = emit(token_text)) {
    return r;
  }
  s->decoded = next;
  return PG_OK;
}

int pg_is_incremental_decode_safe(const char* text, size_t len) {
  return text && decode_safe(std::string(text, len)) ? 1 : 0;
}

int pg_escape_raw_token(const char* token, size_t len, char* out, size_t cap, size_t* out_len) {
  if ((!token && len) || !out_len || (!out && cap)) return set_error(PG_INVALID_INPUT, "null argument");
  std::string esc;
  esc.reserve(len);
  for (size_t i = 0; i < len;) {
    const unsigned char c = (unsigned char)token[i];
    // one UTF-8 scalar: its code point decides, its bytes are copied
    size_t n = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1;
    if (i + n > len) n = 1;
    uint32_t cp = c;
    if (n == 2) cp = ((c & 0x1Fu) << 6) | ((unsigned char)token[i + 1] & 0x3Fu);
    else if (n > 2) cp = 0x10000;  // anything of three or four bytes is no control character
    if (cp == '\\') esc += "\\\\";
    else if (cp == '\t') esc += "\\t";
    else if (cp == '\n') esc += "\\n";
    else if (cp == '\r') esc += "\\r";
    else if (cp < 0x20 || (cp >= 0x7F && cp <= 0x9F)) {  // char::is_control: general category Cc
      char buf[16];
      snprintf(buf, sizeof(buf), "\\u{%x}", cp);
      esc += buf;
    } else {
      esc.append(token + i, n);
    }
    i += n;
  }
  *out_len = esc.size();
  if (esc.size() <= cap && out) memcpy(out, esc.data(), esc.size());
  return PG_OK;
}

uint64_t pg_generation_stats_total_model_tokens(const pg_generation_stats* s) {
  return s ? s->prompt_tokens + s->generated_tokens : 0;
}
double pg_generation_stats_prefill_tokens_per_second(const pg_generation_stats* s) {
  return s ? rate(s->prompt_tokens, s->prefill_time) : 0.0;
}
double pg_generation_stats_decode_tokens_per_second(const pg_generation_stats* s) {
  return s ? rate(s->generated_tokens, s->decode_time) : 0.0;
}
double pg_generation_stats_total_tokens_per_second(const pg_generation_stats* s) {
  return s ? rate(s->prompt_tokens + s->generated_tokens, s->total_generation_time) : 0.0;
}
double pg_generation_stats_average_decode_token_time(const pg_generation_stats* s) {
  if (!s || s->generated_tokens == 0) return -1.0;
  return s->decode_time / (double)s->generated_tokens;
}

}  // extern "C"
