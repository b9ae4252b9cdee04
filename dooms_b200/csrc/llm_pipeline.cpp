#include "llm_pipeline.h"

#include <algorithm>
#include <cctype>
#include <chrono>
#include <climits>
#include <cmath>
#include <numeric>
#include <queue>

#include "unicode_ranges.h"

namespace dooms {

namespace {

template <size_t N> bool in_ranges(const CodePointRange (&ranges)[N], uint32_t cp) {
    size_t lo = 0, hi = N;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (cp > ranges[mid].last) lo = mid + 1;
        else if (cp < ranges[mid].first) hi = mid;
        else return true;
    }
    return false;
}
bool is_letter(uint32_t cp) { return cp < 0x80 ? ((cp | 0x20u) >= 'a' && (cp | 0x20u) <= 'z') : in_ranges(kLetterRanges, cp); }      // \p{L}
bool is_number(uint32_t cp) { return cp < 0x80 ? (cp >= '0' && cp <= '9') : in_ranges(kNumberRanges, cp); }                          // \p{N}
bool is_space(uint32_t cp) {                                                                                                         // \s (White_Space)
    return cp == ' ' || (cp >= 9 && cp <= 13) || cp == 0x85 || cp == 0xA0 || cp == 0x1680 || (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 || cp == 0x2029 ||
           cp == 0x202F || cp == 0x205F || cp == 0x3000;
}

// UTF-8 encoding of a code point.
void put_utf8(std::string & s, uint32_t cp) {
    if (cp < 0x80) s += char(cp);
    else if (cp < 0x800) { s += char(0xC0 | (cp >> 6)); s += char(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { s += char(0xE0 | (cp >> 12)); s += char(0x80 | ((cp >> 6) & 0x3F)); s += char(0x80 | (cp & 0x3F)); }
    else { s += char(0xF0 | (cp >> 18)); s += char(0x80 | ((cp >> 12) & 0x3F)); s += char(0x80 | ((cp >> 6) & 0x3F)); s += char(0x80 | (cp & 0x3F)); }
}
// Code points of a UTF-8 string (malformed bytes pass through as themselves).
std::vector<uint32_t> code_points(const std::string & s) {
    std::vector<uint32_t> out;
    for (size_t i = 0; i < s.size();) {
        const unsigned char c = static_cast<unsigned char>(s[i]);
        const int n = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC0 ? 2 : 1;
        if (n == 1 || i + size_t(n) > s.size()) { out.push_back(c); i++; continue; }
        uint32_t cp = c & (0xFF >> (n + 1));
        for (int k = 1; k < n; k++) cp = (cp << 6) | (static_cast<unsigned char>(s[i + size_t(k)]) & 0x3F);
        out.push_back(cp);
        i += size_t(n);
    }
    return out;
}

// The byte alphabet of byte-level BPE vocabularies (GPT-2's): printable bytes stand for themselves, the other 68 bytes for the code points from U+0100 on.
struct ByteAlphabet {
    uint32_t to_cp[256];
    std::unordered_map<uint32_t, uint8_t> to_byte;
    ByteAlphabet() {
        uint32_t next = 256;
        for (int b = 0; b < 256; b++) {
            const bool printable = (b >= 0x21 && b <= 0x7E) || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
            to_cp[b] = printable ? uint32_t(b) : next++;
            to_byte[to_cp[b]] = uint8_t(b);
        }
    }
};
const ByteAlphabet & alphabet() { static const ByteAlphabet a; return a; }

int32_t int_key(const GgufFile & f, const char * key, int32_t fallback) {
    auto v = f.get_uint(key);
    return v.is_ok() ? int32_t(v.value()) : fallback;
}

// How much of s (from the front) is whole characters: a multi-byte character cut off at the end stays behind.
size_t whole_characters(const std::string & s) {
    for (size_t back = 1; back <= 3 && back <= s.size(); back++) {
        const unsigned char c = static_cast<unsigned char>(s[s.size() - back]);
        if ((c & 0xC0) == 0x80) continue;      // a continuation byte: its lead byte is further back
        const size_t length = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC0 ? 2 : 1;
        return length > back ? s.size() - back : s.size();
    }
    return s.size();
}

using Clock = std::chrono::steady_clock;
double ms_since(Clock::time_point t) { return std::chrono::duration<double, std::milli>(Clock::now() - t).count(); }

}  // namespace

// The words a byte-level BPE vocabulary merges within, as byte ranges of `text`: what the pre-tokenizer regexes of the model families give, matched by
// hand (first alternative that matches at a position wins, as in the regex engines; llama.cpp applies the same patterns for tokenizer.ggml.pre):
//   GPT-2:    's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
//   Llama 3:  (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
//   Qwen2:    the same with \p{N} (one digit) in place of \p{N}{1,3}
std::vector<std::pair<size_t, size_t>> split_words(const std::string & text, int kind) {
    constexpr int kGpt2 = 0, kLlama3 = 1;
    std::vector<uint32_t> cp;
    std::vector<size_t> at;
    for (size_t i = 0; i < text.size();) {
        const unsigned char c = static_cast<unsigned char>(text[i]);
        int n = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC0 ? 2 : 1;
        if (i + size_t(n) > text.size()) n = 1;
        uint32_t v = n == 1 ? c : c & (0xFFu >> (n + 1));
        for (int k = 1; k < n; k++) v = (v << 6) | (static_cast<unsigned char>(text[i + size_t(k)]) & 0x3F);
        cp.push_back(v);
        at.push_back(i);
        i += size_t(n);
    }
    const size_t n = cp.size();
    at.push_back(text.size());
    auto L = [&](size_t k) { return k < n && is_letter(cp[k]); };
    auto N = [&](size_t k) { return k < n && is_number(cp[k]); };
    auto S = [&](size_t k) { return k < n && is_space(cp[k]); };
    auto O = [&](size_t k) { return k < n && !is_space(cp[k]) && !is_letter(cp[k]) && !is_number(cp[k]); };
    auto NL = [&](size_t k) { return k < n && (cp[k] == '\r' || cp[k] == '\n'); };
    auto low = [&](size_t k) -> uint32_t { return k >= n ? 0u : (kind != kGpt2 && cp[k] >= 'A' && cp[k] <= 'Z') ? cp[k] + 32u : cp[k]; };
    std::vector<std::pair<size_t, size_t>> words;
    for (size_t i = 0; i < n;) {
        size_t j = 0;
        if (cp[i] == '\'') {      // a contraction
            const uint32_t a = low(i + 1), b = low(i + 2);
            if (a == 's' || a == 't' || a == 'm' || a == 'd') j = i + 2;
            else if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) j = i + 3;
        }
        if (!j) {                  // letters, with the one character allowed in front of them
            const bool lead = kind == kGpt2 ? cp[i] == ' ' : (!NL(i) && !L(i) && !N(i));
            const size_t k = (lead && L(i + 1)) ? i + 1 : i;
            if (L(k)) { j = k; while (L(j)) j++; }
        }
        if (!j) {                  // digits
            if (kind == kGpt2) {
                const size_t k = (cp[i] == ' ' && N(i + 1)) ? i + 1 : i;
                if (N(k)) { j = k; while (N(j)) j++; }
            } else if (N(i)) {
                j = i + 1;
                if (kind == kLlama3) while (N(j) && j - i < 3) j++;
            }
        }
        if (!j) {                  // anything else that is no space, with a space in front (and, outside GPT-2, the line breaks behind)
            const size_t k = (cp[i] == ' ' && O(i + 1)) ? i + 1 : i;
            if (O(k)) {
                j = k;
                while (O(j)) j++;
                if (kind != kGpt2) while (NL(j)) j++;
            }
        }
        if (!j && S(i)) {
            size_t e = i;
            while (S(e)) e++;
            if (kind != kGpt2) {   // up to the last line break of the run
                for (size_t k = e; k > i; k--) if (NL(k - 1)) { j = k; break; }
            }
            if (!j) j = (e == n || e - i == 1) ? e : e - 1;      // the run, short of its last character when a word follows (that one goes with the word)
        }
        if (!j) j = i + 1;
        words.emplace_back(at[i], at[j]);
        i = j;
    }
    return words;
}

// ---------------------------------------------------------------- vocabulary

Result<Vocab> Vocab::from_gguf(const GgufFile & file) {
    const auto & md = file.metadata();
    const auto tokens = md.find("tokenizer.ggml.tokens");
    if (tokens == md.end() || tokens->second.type != GgufValueType::Array || tokens->second.element_type != GgufValueType::String) {
        return invalid_argument("the model file has no tokenizer.ggml.tokens (an array of strings)");
    }
    auto model = file.get_string("tokenizer.ggml.model");
    const std::string kind = model.is_ok() ? model.value() : "llama";
    if (kind != "gpt2" && kind != "llama") return unsupported("tokenizer model '" + kind + "': byte-level BPE (gpt2) and sentencepiece pieces (llama) are read");
    Vocab v;
    v.byte_level_ = kind == "gpt2";
    if (auto pre = file.get_string("tokenizer.ggml.pre"); pre.is_ok()) {
        const std::string & name = pre.value();
        if (name == "llama-bpe" || name == "llama3" || name == "llama-v3") { v.pre_ = 1; v.ignore_merges_ = true; }
        else if (name == "qwen2" || name == "deepseek-r1-qwen") v.pre_ = 2;
    }
    const size_t n = tokens->second.items.size();
    v.raw_.reserve(n);
    for (const GgufValue & t : tokens->second.items) v.raw_.push_back(t.s);
    v.special_.assign(n, false);
    if (const auto types = md.find("tokenizer.ggml.token_type"); types != md.end() && types->second.items.size() == n) {
        // 3 = control, 4 = user defined: no text of their own in the answer (6 = byte: handled as a piece)
        for (size_t i = 0; i < n; i++) {
            const int64_t t = types->second.items[i].i;
            v.special_[i] = t == 3;
            if ((t == 3 || t == 4) && !v.raw_[i].empty()) v.marked_.emplace_back(v.raw_[i], int32_t(i));
        }
        std::stable_sort(v.marked_.begin(), v.marked_.end(), [](const auto & a, const auto & b) { return a.first.size() > b.first.size(); });
    }
    if (auto tmpl = file.get_string("tokenizer.chat_template"); tmpl.is_ok()) v.chat_template_ = tmpl.value();
    v.pieces_.resize(n);
    for (size_t i = 0; i < n; i++) {
        const std::string & raw = v.raw_[i];
        v.ids_.emplace(raw, int32_t(i));
        if (v.special_[i]) continue;
        std::string & out = v.pieces_[i];
        if (v.byte_level_) {
            for (uint32_t cp : code_points(raw)) {
                const auto b = alphabet().to_byte.find(cp);
                if (b != alphabet().to_byte.end()) out += char(b->second);
                else put_utf8(out, cp);
            }
        } else if (raw.size() == 6 && raw.compare(0, 3, "<0x") == 0 && raw[5] == '>') {
            out = std::string(1, char(std::stoi(raw.substr(3, 2), nullptr, 16)));
        } else {
            for (uint32_t cp : code_points(raw)) { if (cp == 0x2581) out += ' '; else put_utf8(out, cp); }
        }
    }
    if (const auto merges = md.find("tokenizer.ggml.merges"); merges != md.end()) {
        int32_t rank = 0;
        for (const GgufValue & m : merges->second.items) v.merge_rank_.emplace(m.s, rank++);
    }
    if (const auto scores = md.find("tokenizer.ggml.scores"); scores != md.end() && scores->second.items.size() == n) {
        v.scores_.resize(n);
        for (size_t i = 0; i < n; i++) v.scores_[i] = float(scores->second.items[i].f);
    }
    v.bos_ = int_key(file, "tokenizer.ggml.bos_token_id", -1);
    for (const char * key : {"tokenizer.ggml.eos_token_id", "tokenizer.ggml.eot_token_id", "tokenizer.ggml.eom_token_id"}) {
        const int32_t id = int_key(file, key, -1);
        if (id >= 0 && std::find(v.eog_.begin(), v.eog_.end(), id) == v.eog_.end()) v.eog_.push_back(id);
    }
    auto add_bos = file.get_bool("tokenizer.ggml.add_bos_token");
    v.add_bos_ = add_bos.is_ok() ? add_bos.value() : !v.byte_level_;      // sentencepiece models ask for it unless they say otherwise
    auto space_prefix = file.get_bool("tokenizer.ggml.add_space_prefix");
    v.space_prefix_ = space_prefix.is_ok() ? space_prefix.value() : true;
    return v;
}

const std::string & Vocab::piece(int32_t id) const {
    static const std::string none;
    return id >= 0 && id < size() ? pieces_[size_t(id)] : none;
}

bool Vocab::is_end_of_generation(int32_t id) const { return std::find(eog_.begin(), eog_.end(), id) != eog_.end(); }

Result<std::vector<int32_t>> Vocab::tokenize(const std::string & text, bool add_special, bool parse_special) const {
    if (text.empty()) return invalid_argument("tokenize: empty text");
    std::vector<int32_t> out;
    if (add_special && add_bos_ && bos_ >= 0) out.push_back(bos_);
    // the text in stretches between marked tokens; a sentencepiece stretch gets its space in front at the start and after a marked token
    size_t from = 0, at = 0;
    bool after_marked = true;
    auto flush = [&](size_t end) -> Status {
        if (end > from) {
            Status s = tokenize_plain(text.substr(from, end - from), after_marked, &out);
            if (!s.is_ok()) return s;
            after_marked = false;
        }
        return Status();
    };
    while (at < text.size() && !marked_.empty()) {
        const std::pair<std::string, int32_t> * hit = nullptr;
        for (const auto & m : marked_) {
            if (!parse_special && special_[size_t(m.second)]) continue;
            if (text.compare(at, m.first.size(), m.first) == 0) { hit = &m; break; }
        }
        if (!hit) { at++; continue; }
        Status s = flush(at);
        if (!s.is_ok()) return s;
        out.push_back(hit->second);
        after_marked = true;
        at += hit->first.size();
        from = at;
    }
    Status s = flush(text.size());
    if (!s.is_ok()) return s;
    return out;
}

Status Vocab::tokenize_plain(const std::string & text, bool space_in_front, std::vector<int32_t> * result) const {
    std::vector<int32_t> & out = *result;
    if (!byte_level_) {
        // sentencepiece: the escaped text as a chain of characters; the pair whose concatenation is the best-scoring piece is merged until none is a piece
        std::string escaped = (space_in_front && space_prefix_) ? "\xE2\x96\x81" : "";
        for (char c : text) { if (c == ' ') escaped += "\xE2\x96\x81"; else escaped += c; }
        struct Sym { size_t at, len; int prev, next; };
        std::vector<Sym> sym;
        for (size_t i = 0; i < escaped.size();) {
            const unsigned char c = static_cast<unsigned char>(escaped[i]);
            size_t len = c < 0x80 ? 1 : c < 0xE0 ? 2 : c < 0xF0 ? 3 : 4;
            len = std::min(len, escaped.size() - i);
            sym.push_back({i, len, int(sym.size()) - 1, int(sym.size()) + 1});
            i += len;
        }
        if (!sym.empty()) sym.back().next = -1;
        // candidate pairs in a heap: best score first, leftmost on ties; a popped pair counts only if both halves still have the lengths it was made with
        struct Pair { float score; int left, right; size_t left_len, right_len; };
        auto worse = [](const Pair & a, const Pair & b) { return a.score != b.score ? a.score < b.score : a.left > b.left; };
        std::priority_queue<Pair, std::vector<Pair>, decltype(worse)> heap(worse);
        auto offer = [&](int i, int j) {
            if (i < 0 || j < 0) return;
            const Sym & a = sym[size_t(i)], & b = sym[size_t(j)];
            const auto id = ids_.find(escaped.substr(a.at, a.len + b.len));
            if (id == ids_.end()) return;
            heap.push({size_t(id->second) < scores_.size() ? scores_[size_t(id->second)] : 0.f, i, j, a.len, b.len});
        };
        for (int i = 0; i + 1 < int(sym.size()); i++) offer(i, i + 1);
        while (!heap.empty()) {
            const Pair top = heap.top();
            heap.pop();
            Sym & a = sym[size_t(top.left)];
            Sym & b = sym[size_t(top.right)];
            if (a.len != top.left_len || b.len != top.right_len || a.next != top.right) continue;      // one of them was merged meanwhile
            a.len += b.len;
            a.next = b.next;
            b.len = 0;
            if (b.next >= 0) sym[size_t(b.next)].prev = top.left;
            offer(a.prev, top.left);
            offer(top.left, a.next);
        }
        for (int i = sym.empty() ? -1 : 0; i >= 0; i = sym[size_t(i)].next) {
            const std::string piece = escaped.substr(sym[size_t(i)].at, sym[size_t(i)].len);
            const auto id = ids_.find(piece);
            if (id != ids_.end()) { out.push_back(id->second); continue; }
            for (unsigned char c : piece) {
                char name[8];
                snprintf(name, sizeof name, "<0x%02X>", unsigned(c));
                const auto b = ids_.find(name);
                if (b == ids_.end()) return invalid_argument("tokenize: the vocabulary has no token for a byte of the text");
                out.push_back(b->second);
            }
        }
        return Status();
    }
    for (const auto & [at, end] : split_words(text, pre_)) {
        // the word's bytes in the byte alphabet, then merges by rank
        std::vector<std::string> sym;
        for (size_t i = at; i < end; i++) { std::string s; put_utf8(s, alphabet().to_cp[static_cast<unsigned char>(text[i])]); sym.push_back(std::move(s)); }
        if (ignore_merges_) {      // Llama 3 vocabularies: a word that is a token goes out as that token, whatever the merges would build
            std::string whole;
            for (const std::string & s : sym) whole += s;
            if (const auto id = ids_.find(whole); id != ids_.end()) { out.push_back(id->second); continue; }
        }
        while (sym.size() > 1) {
            int32_t best = INT32_MAX;
            size_t where = 0;
            for (size_t i = 0; i + 1 < sym.size(); i++) {
                const auto r = merge_rank_.find(sym[i] + " " + sym[i + 1]);
                if (r != merge_rank_.end() && r->second < best) { best = r->second; where = i; }
            }
            if (best == INT32_MAX) break;
            sym[where] += sym[where + 1];
            sym.erase(sym.begin() + long(where) + 1);
        }
        for (const std::string & s : sym) {
            const auto id = ids_.find(s);
            if (id != ids_.end()) { out.push_back(id->second); continue; }
            for (uint32_t cp : code_points(s)) {      // a symbol the vocabulary lacks: its bytes one by one
                std::string one;
                put_utf8(one, cp);
                const auto b = ids_.find(one);
                if (b == ids_.end()) return invalid_argument("tokenize: the vocabulary has no token for a byte of the text");
                out.push_back(b->second);
            }
        }
    }
    return Status();
}

// The families below are the ones llama.cpp's llama_chat_apply_template knows by these markers; their formats are the model cards' own.
Result<std::string> Vocab::apply_chat_template(const std::vector<ChatMessage> & messages, bool add_generation_prompt) const {
    if (messages.empty()) return invalid_argument("no messages");
    for (const ChatMessage & m : messages) if (m.role.empty()) return invalid_argument("a message has an empty role");
    if (chat_template_.empty()) return unsupported("the model file has no chat template");
    auto has = [&](const char * marker) { return chat_template_.find(marker) != std::string::npos; };
    auto trimmed = [](const std::string & t) {
        size_t a = 0, b = t.size();
        while (a < b && std::isspace(static_cast<unsigned char>(t[a]))) a++;
        while (b > a && std::isspace(static_cast<unsigned char>(t[b - 1]))) b--;
        return t.substr(a, b - a);
    };
    std::string out;
    if (has("<|im_start|>") && has("<end_of_utterance>")) {          // SmolVLM: "User: ...<end_of_utterance>\nAssistant:"
        out = "<|im_start|>";
        for (const ChatMessage & m : messages) {
            if (m.role == "system") out += m.content + "\n\n";
            else out += (m.role == "user" ? "User: " : "Assistant: ") + m.content + "<end_of_utterance>\n";
        }
        if (add_generation_prompt) out += "Assistant:";
    } else if (has("<|im_start|>") && !has("<|im_sep|>")) {          // ChatML (Qwen2 and many others)
        for (const ChatMessage & m : messages) out += "<|im_start|>" + m.role + "\n" + m.content + "<|im_end|>\n";
        if (add_generation_prompt) out += "<|im_start|>assistant\n";
    } else if (has("<|start_header_id|>") && has("<|end_header_id|>")) {      // Llama 3
        for (const ChatMessage & m : messages) out += "<|start_header_id|>" + m.role + "<|end_header_id|>\n\n" + trimmed(m.content) + "<|eot_id|>";
        if (add_generation_prompt) out += "<|start_header_id|>assistant<|end_header_id|>\n\n";
    } else {
        return unsupported("this model's chat template is of a family this library does not know (ChatML, Llama 3 and SmolVLM are written)");
    }
    return out;
}

// ---------------------------------------------------------------- sampler

Result<Sampler> Sampler::create(const SamplerOptions & o) {
    if (!(o.temperature >= 0.f) || !(o.top_p > 0.f && o.top_p <= 1.f) || o.top_k < 0 || !(o.repeat_penalty > 0.f)) {
        return invalid_argument("sampler: temperature >= 0, top_p in (0, 1], top_k >= 0 and repeat_penalty > 0 are required");
    }
    Sampler s;
    s.o_ = o;
    s.state_ = 0x9E3779B97F4A7C15ull ^ (uint64_t(o.seed) * 0xD1342543DE82EF95ull);
    return s;
}

double Sampler::uniform() {      // splitmix64
    uint64_t z = (state_ += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return double(z >> 11) * (1.0 / 9007199254740992.0);
}

void Sampler::accept(int32_t token) {
    recent_.push_back(token);
    if (recent_.size() > 64) recent_.erase(recent_.begin());
}

int32_t Sampler::sample(const float * logits, int32_t n) {
    std::vector<std::pair<float, int32_t>> cand;
    cand.reserve(size_t(n));
    for (int32_t i = 0; i < n; i++) if (logits[i] == logits[i]) cand.emplace_back(logits[i], i);      // NaN never wins
    if (cand.empty()) { accept(0); return 0; }
    if (o_.repeat_penalty != 1.f) {
        for (auto & c : cand) {
            if (std::find(recent_.begin(), recent_.end(), c.second) != recent_.end()) c.first = c.first > 0 ? c.first / o_.repeat_penalty : c.first * o_.repeat_penalty;
        }
    }
    auto by_logit = [](const std::pair<float, int32_t> & a, const std::pair<float, int32_t> & b) { return a.first > b.first || (a.first == b.first && a.second < b.second); };
    int32_t chosen;
    if (o_.temperature == 0.f) {
        chosen = std::min_element(cand.begin(), cand.end(), by_logit)->second;      // the largest logit, lowest index on ties
    } else {
        const size_t keep = o_.top_k > 0 ? std::min(size_t(o_.top_k), cand.size()) : cand.size();
        std::partial_sort(cand.begin(), cand.begin() + long(keep), cand.end(), by_logit);
        cand.resize(keep);
        // the order of the reference's chain (src/models/vlm/text_decoder.cpp:239-242): top-k, then top-p on the probabilities at temperature 1, then the
        // temperature, then the draw
        std::vector<double> p(keep);
        const double top = cand[0].first;
        size_t last = keep;
        if (o_.top_p < 1.f) {      // the smallest prefix whose probability reaches top_p
            double total = 0, acc = 0;
            for (size_t i = 0; i < keep; i++) { p[i] = std::exp(double(cand[i].first) - top); total += p[i]; }
            for (size_t i = 0; i < keep; i++) { acc += p[i] / total; if (acc >= double(o_.top_p)) { last = i + 1; break; } }
        }
        for (size_t i = 0; i < last; i++) p[i] = std::exp((double(cand[i].first) - top) / double(o_.temperature));
        double mass = 0;
        for (size_t i = 0; i < last; i++) mass += p[i];
        double u = uniform() * mass;
        size_t pick = last - 1;
        for (size_t i = 0; i < last; i++) { if (u < p[i]) { pick = i; break; } u -= p[i]; }
        chosen = cand[pick].second;
    }
    accept(chosen);
    return chosen;
}

// ---------------------------------------------------------------- text stream

TextStream::TextStream(const Vocab & vocab, const std::vector<std::string> & stops, std::function<bool(const std::string &)> on_text, LlmGeneration * out)
    : vocab_(vocab), stops_(stops), on_text_(std::move(on_text)), out_(*out) {}

bool TextStream::release(size_t n) {
    if (n == 0) return true;
    const std::string piece = held_.substr(0, n);
    held_.erase(0, n);
    out_.text += piece;
    return !on_text_ || on_text_(piece);
}

bool TextStream::push(int32_t token) {
    out_.tokens.push_back(token);
    if (vocab_.is_end_of_generation(token)) { out_.stopped = true; return false; }
    held_ += vocab_.piece(token);
    // a stop string inside what is held: the text ends right before the earliest one
    size_t cut = std::string::npos;
    for (const std::string & s : stops_) cut = std::min(cut, held_.find(s));
    if (cut != std::string::npos) {
        held_.resize(cut);
        if (release(held_.size())) out_.stopped = true;
        else out_.cancelled = true;
        return false;
    }
    // hold back the longest tail that could still grow into a stop string, and a character that is not whole yet
    size_t keep = 0;
    for (const std::string & s : stops_) {
        for (size_t k = std::min(s.size() - 1, held_.size()); k > keep; k--) {
            if (held_.compare(held_.size() - k, k, s, 0, k) == 0) { keep = k; break; }
        }
    }
    const size_t ready = std::min(held_.size() - keep, whole_characters(held_));
    if (!release(ready)) { out_.cancelled = true; return false; }
    return true;
}

void TextStream::finish() {
    const bool ended_by_token = out_.stopped && !out_.tokens.empty() && vocab_.is_end_of_generation(out_.tokens.back());
    if ((!out_.stopped && !out_.cancelled) || ended_by_token) (void)release(held_.size());      // nothing follows that could complete a stop string
}

// ---------------------------------------------------------------- Llm

Result<std::unique_ptr<Llm>> Llm::load(const std::string & path, const LlmOptions & o) {
    NativeLlamaOptions n;
    n.n_ctx = o.n_ctx;
    n.n_batch = o.n_batch;
    auto dec = load_native_llama(path, n, o.cuda);
    if (!dec.is_ok()) return dec.status();
    auto file = GgufFile::open(path);
    if (!file.is_ok()) return file.status();
    auto vocab = Vocab::from_gguf(file.value());
    if (!vocab.is_ok()) return vocab.status();
    if (vocab.value().size() != dec.value()->config().n_vocab) return invalid_argument("the vocabulary's size differs from the embedding table's rows");
    return std::unique_ptr<Llm>(new Llm(std::move(dec).value(), std::move(vocab).value(), std::max(1, o.queue_depth)));
}

Result<LlmGeneration> Llm::generate(const std::string & prompt, const LlmGenerateOptions & o, const std::function<bool(const std::string &)> & on_text, LlmTimings * timings) {
    auto tokens = tokenize(prompt, true);
    if (!tokens.is_ok()) return tokens.status();
    return generate_tokens(tokens.value(), o, on_text, timings);
}

Result<std::vector<int32_t>> Llm::chat_tokens(const std::vector<ChatMessage> & messages) const {
    auto text = vocab_.apply_chat_template(messages, true);
    if (!text.is_ok()) return text.status();
    return vocab_.tokenize(text.value(), /*add_special=*/false, /*parse_special=*/true);
}

Result<LlmGeneration> Llm::chat(const std::vector<ChatMessage> & messages, const LlmGenerateOptions & o, const std::function<bool(const std::string &)> & on_text,
                                LlmTimings * timings) {
    auto tokens = chat_tokens(messages);
    if (!tokens.is_ok()) return tokens.status();
    return generate_tokens(tokens.value(), o, on_text, timings);
}

Result<LlmGeneration> Llm::generate_tokens(const std::vector<int32_t> & prompt, const LlmGenerateOptions & o, const std::function<bool(const std::string &)> & on_text,
                                           LlmTimings * timings) {
    const int32_t n_ctx = context_size();
    if (prompt.empty()) return invalid_argument("generate: empty prompt");
    if (o.max_new_tokens < 1 || o.max_new_tokens >= n_ctx) return invalid_argument("generate: max_new_tokens has to lie in [1, context size)");
    if (std::any_of(o.stop.begin(), o.stop.end(), [](const std::string & s) { return s.empty(); })) return invalid_argument("generate: an empty stop string");
    if (int64_t(prompt.size()) + o.max_new_tokens > n_ctx) {
        return resource_exhausted("generate: " + std::to_string(prompt.size()) + " prompt tokens and " + std::to_string(o.max_new_tokens) + " new ones do not fit the context of " +
                                  std::to_string(n_ctx));
    }
    auto sampler = Sampler::create(o.sampler);
    if (!sampler.is_ok()) return sampler.status();
    const auto t0 = Clock::now();
    LlmTimings tm;
    tm.prompt_tokens = int64_t(prompt.size());
    decoder_->reset();
    DOOMS_RETURN_IF_ERROR(decoder_->eval_tokens(prompt));
    LlmGeneration out;
    TextStream stream(vocab_, o.stop, on_text, &out);
    auto t_decode = t0;
    auto count = [&] {
        // the first token exists once the prompt has gone through the model: its arrival marks the end of the prefill
        if (tm.generated_tokens++ == 0) { tm.prefill_ms = tm.first_token_ms = ms_since(t0); t_decode = Clock::now(); }
    };
    if (sampler.value().greedy()) {
        // the token is picked on the device and the next step reads it there: steps stay queued ahead of the host
        DOOMS_RETURN_IF_ERROR(decoder_->generate(o.max_new_tokens, depth_, [&](int32_t token) { count(); return stream.push(token); }));
    } else {
        for (int32_t i = 0; i < o.max_new_tokens; i++) {
            auto logits = decoder_->logits();
            if (!logits.is_ok()) return logits.status();
            const int32_t token = sampler.value().sample(logits.value().data(), int32_t(logits.value().size()));
            count();
            if (!stream.push(token)) break;
            if (i + 1 < o.max_new_tokens) DOOMS_RETURN_IF_ERROR(decoder_->eval_tokens(&token, 1));
        }
    }
    stream.finish();
    tm.decode_ms = tm.generated_tokens > 1 ? ms_since(t_decode) : 0.0;
    if (timings) *timings = tm;
    return out;
}

Result<LlmGeneration> Llm::generate_from_embeddings(const std::vector<int32_t> & before, const float * image, int32_t image_rows, const std::vector<int32_t> & after,
                                                    int32_t max_new_tokens, const std::function<bool(const std::string &)> & on_text, LlmTimings * timings) {
    const int32_t n_ctx = context_size();
    const size_t E = size_t(decoder_->config().n_embd);
    const size_t rows = before.size() + size_t(std::max(image_rows, 0)) + after.size();
    if (rows == 0 || image_rows < 0 || (image_rows > 0 && image == nullptr)) return invalid_argument("generate_from_embeddings: no rows to evaluate");
    if (max_new_tokens < 1 || max_new_tokens >= n_ctx) return invalid_argument("generate_from_embeddings: max_new_tokens has to lie in [1, context size)");
    if (int64_t(rows) + max_new_tokens > n_ctx) {
        return resource_exhausted("generate_from_embeddings: " + std::to_string(rows) + " rows and " + std::to_string(max_new_tokens) + " new tokens do not fit the context of " +
                                  std::to_string(n_ctx));
    }
    const auto t0 = Clock::now();
    std::vector<float> all(rows * E);
    if (!before.empty()) DOOMS_RETURN_IF_ERROR(decoder_->embed_tokens(before.data(), int32_t(before.size()), all.data()));
    if (image_rows > 0) std::copy(image, image + size_t(image_rows) * E, all.begin() + long(before.size() * E));
    if (!after.empty()) DOOMS_RETURN_IF_ERROR(decoder_->embed_tokens(after.data(), int32_t(after.size()), all.data() + (before.size() + size_t(image_rows)) * E));
    LlmTimings tm;
    tm.prompt_tokens = int64_t(rows);
    decoder_->reset();
    DOOMS_RETURN_IF_ERROR(decoder_->eval_embeddings(all.data(), int32_t(rows)));
    LlmGeneration out;
    static const std::vector<std::string> no_stops;
    TextStream stream(vocab_, no_stops, on_text, &out);
    auto t_decode = t0;
    DOOMS_RETURN_IF_ERROR(decoder_->generate(max_new_tokens, depth_, [&](int32_t token) {
        if (tm.generated_tokens++ == 0) { tm.prefill_ms = tm.first_token_ms = ms_since(t0); t_decode = Clock::now(); }
        return stream.push(token);
    }));
    stream.finish();
    tm.decode_ms = tm.generated_tokens > 1 ? ms_since(t_decode) : 0.0;
    if (timings) *timings = tm;
    return out;
}

}  // namespace dooms
