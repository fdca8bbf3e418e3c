// Tokenizer for the chatbots' text side: reads a Hugging Face tokenizer.json and encodes / decodes as the reference's
// runtime does through the `tokenizers` crate (crates/tl_runtime/src/tokenizer.rs:16-246: tl_tokenizer_new, _encode,
// _decode, _encode_chat, _encode_chat_zephyr).  Host code only.  Two model styles are covered, the two the reference's
// programs load:
//   * byte-level BPE (Llama-3): no normalizer; pre-tokenizer = Split(regex, isolated) + ByteLevel(no prefix space); every
//     byte of a piece becomes one printable code point (the GPT-2 table) and the merges run over those; `ignore_merges`
//     lets a whole piece that is in the vocabulary through unmerged.  The split pattern is matched by a hand-written
//     scanner for the two patterns in use (Llama-3's and GPT-2's); another pattern is refused.
//   * SentencePiece-style BPE (TinyLlama / Llama-2): normalizer Prepend("▁") + Replace(" ", "▁"), no pre-tokenizer, the
//     merges run over the code points of a whole segment, characters outside the vocabulary fall back to their UTF-8
//     bytes as <0xHH> tokens (or the unknown token, consecutive ones fused).
// Added tokens (special ones included) are cut out of the text first, leftmost-longest, and keep their ids.
// The merge loop is the crate's: all adjacent pairs in a heap ordered by (merge rank, position); pop, merge if both
// halves are still what they were, push the new neighbours.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <queue>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "tlb_internal.h"

namespace tlb {
namespace {

#include "unicode_ln.inc"

// ---------------------------------------------------------------- a small JSON reader
struct JVal {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal *get(const char *key) const
    {
        for (auto &kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is(Kind k) const { return kind == k; }
};

void put_utf8(std::string &s, uint32_t cp)
{
    if (cp < 0x80) s += (char)cp;
    else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
    else { s += (char)(0xF0 | (cp >> 18)); s += (char)(0x80 | ((cp >> 12) & 0x3F)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
}

struct JReader {
    const char *p, *end;
    bool ok = true;
    int depth = 0;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) p++; }
    bool lit(const char *s) { size_t n = strlen(s); if ((size_t)(end - p) >= n && !memcmp(p, s, n)) { p += n; return true; } return false; }
    int hex4()
    {
        if (end - p < 4) return -1;
        int v = 0;
        for (int i = 0; i < 4; i++) {
            char c = p[i];
            int d = c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : -1;
            if (d < 0) return -1;
            v = v * 16 + d;
        }
        p += 4;
        return v;
    }
    bool string(std::string &out)
    {
        if (p >= end || *p != '"') return false;
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return false;
                char c = *p++;
                switch (c) {
                    case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break; case 'f': out += '\f'; break;
                    case 'u': {
                        int hi = hex4();
                        if (hi < 0) return false;
                        uint32_t cp = (uint32_t)hi;
                        if (hi >= 0xD800 && hi < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {   // surrogate pair
                            p += 2;
                            int lo = hex4();
                            if (lo < 0xDC00 || lo > 0xDFFF) return false;
                            cp = 0x10000 + (((uint32_t)hi - 0xD800) << 10) + ((uint32_t)lo - 0xDC00);
                        }
                        put_utf8(out, cp);
                        break;
                    }
                    default: out += c;   // \" \\ \/
                }
            } else out += *p++;
        }
        if (p >= end) return false;
        p++;
        return true;
    }
    bool value(JVal &v)
    {
        if (++depth > 64) return false;
        ws();
        bool r = false;
        if (p >= end) r = false;
        else if (*p == '{') {
            p++;
            v.kind = JVal::OBJ;
            ws();
            if (p < end && *p == '}') { p++; r = true; }
            else for (;;) {
                ws();
                std::string k;
                if (!string(k)) break;
                ws();
                if (p >= end || *p++ != ':') break;
                v.obj.emplace_back(std::move(k), JVal());
                if (!value(v.obj.back().second)) break;
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; r = true; }
                break;
            }
        } else if (*p == '[') {
            p++;
            v.kind = JVal::ARR;
            ws();
            if (p < end && *p == ']') { p++; r = true; }
            else for (;;) {
                v.arr.emplace_back();
                if (!value(v.arr.back())) break;
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; r = true; }
                break;
            }
        } else if (*p == '"') { v.kind = JVal::STR; r = string(v.str); }
        else if (lit("true")) { v.kind = JVal::BOOL; v.b = true; r = true; }
        else if (lit("false")) { v.kind = JVal::BOOL; v.b = false; r = true; }
        else if (lit("null")) { v.kind = JVal::NUL; r = true; }
        else {
            char *e = nullptr;
            v.num = strtod(p, &e);
            if (e && e > p && e <= end) { v.kind = JVal::NUM; p = e; r = true; }
        }
        depth--;
        return r;
    }
};

// ---------------------------------------------------------------- code points
bool in_ranges(const uint32_t (*t)[2], size_t n, uint32_t cp)
{
    size_t lo = 0, hi = n;
    while (lo < hi) {
        size_t mid = (lo + hi) / 2;
        if (cp < t[mid][0]) hi = mid;
        else if (cp > t[mid][1]) lo = mid + 1;
        else return true;
    }
    return false;
}
bool is_L(uint32_t cp) { return in_ranges(kUnicodeL, sizeof(kUnicodeL) / sizeof(kUnicodeL[0]), cp); }
bool is_N(uint32_t cp) { return in_ranges(kUnicodeN, sizeof(kUnicodeN) / sizeof(kUnicodeN[0]), cp); }
bool is_S(uint32_t cp)   // \s: the White_Space property
{
    return (cp >= 9 && cp <= 13) || cp == 0x20 || cp == 0x85 || cp == 0xA0 || cp == 0x1680 || (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 ||
           cp == 0x2029 || cp == 0x202F || cp == 0x205F || cp == 0x3000;
}
bool is_nl(uint32_t cp) { return cp == '\r' || cp == '\n'; }

// text -> code points with their byte offsets (malformed bytes become U+FFFD, one per byte, as a lossy conversion gives)
void decode_utf8(const std::string &s, std::vector<uint32_t> &cps, std::vector<uint32_t> &offs)
{
    size_t i = 0, n = s.size();
    while (i < n) {
        unsigned char c = (unsigned char)s[i];
        uint32_t cp = 0xFFFD;
        int len = 1;
        if (c < 0x80) cp = c;
        else if ((c >> 5) == 6 && i + 1 < n && ((unsigned char)s[i + 1] >> 6) == 2) { cp = ((c & 31u) << 6) | ((unsigned char)s[i + 1] & 63u); len = 2; if (cp < 0x80) { cp = 0xFFFD; len = 1; } }
        else if ((c >> 4) == 14 && i + 2 < n && ((unsigned char)s[i + 1] >> 6) == 2 && ((unsigned char)s[i + 2] >> 6) == 2) {
            cp = ((c & 15u) << 12) | (((unsigned char)s[i + 1] & 63u) << 6) | ((unsigned char)s[i + 2] & 63u); len = 3;
            if (cp < 0x800 || (cp >= 0xD800 && cp <= 0xDFFF)) { cp = 0xFFFD; len = 1; }
        } else if ((c >> 3) == 30 && i + 3 < n && ((unsigned char)s[i + 1] >> 6) == 2 && ((unsigned char)s[i + 2] >> 6) == 2 && ((unsigned char)s[i + 3] >> 6) == 2) {
            cp = ((c & 7u) << 18) | (((unsigned char)s[i + 1] & 63u) << 12) | (((unsigned char)s[i + 2] & 63u) << 6) | ((unsigned char)s[i + 3] & 63u); len = 4;
            if (cp < 0x10000 || cp > 0x10FFFF) { cp = 0xFFFD; len = 1; }
        }
        cps.push_back(cp);
        offs.push_back((uint32_t)i);
        i += len;
    }
    offs.push_back((uint32_t)n);
}

// ---------------------------------------------------------------- the split patterns
enum Pattern { PAT_NONE = 0, PAT_LLAMA3 = 1, PAT_GPT2 = 2 };
const char *kLlama3Pattern = "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}{1,3}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+";
const char *kGpt2Pattern = "'s|'t|'re|'ve|'m|'ll|'d| ?\\p{L}+| ?\\p{N}+| ?[^\\s\\p{L}\\p{N}]+|\\s+(?!\\S)|\\s+";

// Length (in code points) of the match of the pattern at position i (leftmost alternative that matches, greedy inside, with
// the back-tracking the alternatives need); 0: no alternative matches there (the code point then stands alone).
size_t match_at(Pattern pat, const std::vector<uint32_t> &c, size_t i)
{
    const size_t n = c.size();
    auto lower = [](uint32_t x) { return x >= 'A' && x <= 'Z' ? x + 32 : x; };
    // contractions
    if (c[i] == '\'' && i + 1 < n) {
        const uint32_t a = pat == PAT_LLAMA3 ? lower(c[i + 1]) : c[i + 1];
        const uint32_t b = i + 2 < n ? (pat == PAT_LLAMA3 ? lower(c[i + 2]) : c[i + 2]) : 0;
        if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
    }
    auto run = [&](size_t from, bool (*pred)(uint32_t)) { size_t j = from; while (j < n && pred(c[j])) j++; return j; };
    auto other = [](uint32_t x) { return !is_S(x) && !is_L(x) && !is_N(x); };
    if (pat == PAT_LLAMA3) {
        // [^\r\n\p{L}\p{N}]?\p{L}+
        if (!is_nl(c[i]) && !is_L(c[i]) && !is_N(c[i]) && i + 1 < n && is_L(c[i + 1])) return run(i + 1, is_L) - i;
        if (is_L(c[i])) return run(i, is_L) - i;
        // \p{N}{1,3}
        if (is_N(c[i])) { size_t j = i; while (j < n && j < i + 3 && is_N(c[j])) j++; return j - i; }
        // " ?[^\s\p{L}\p{N}]+[\r\n]*"
        {
            size_t j = i;
            if (c[j] == ' ' && j + 1 < n && other(c[j + 1])) j++;
            if (other(c[j])) {
                j = run(j, other);
                j = run(j, is_nl);
                return j - i;
            }
        }
    } else {
        // " ?\p{L}+", " ?\p{N}+", " ?[^\s\p{L}\p{N}]+"
        size_t j = i;
        if (c[j] == ' ' && j + 1 < n && !is_S(c[j + 1])) j++;
        if (is_L(c[j])) return run(j, is_L) - i;
        if (is_N(c[j])) return run(j, is_N) - i;
        if (other(c[j])) return run(j, other) - i;
    }
    if (is_S(c[i])) {
        const size_t e = run(i, is_S);
        if (pat == PAT_LLAMA3) {   // \s*[\r\n]+ : up to the last line break of the white-space run
            size_t last = n;
            for (size_t j = i; j < e; j++)
                if (is_nl(c[j])) last = j;
            if (last != n) return last + 1 - i;
        }
        // \s+(?!\S): all of the run if the text ends there, else all but its last code point (if that leaves any)
        if (e == n) return e - i;
        if (e - i >= 2) return e - 1 - i;
        return 1;   // \s+
    }
    return 0;
}

// ---------------------------------------------------------------- the tokenizer
struct PairHash {
    size_t operator()(const std::pair<int, int> &p) const { return std::hash<uint64_t>()(((uint64_t)(uint32_t)p.first << 32) | (uint32_t)p.second); }
};

}  // namespace
}  // namespace tlb

struct tlb_tokenizer {
    std::vector<std::string> id_to_token;
    std::unordered_map<std::string, int> token_to_id;
    std::unordered_map<std::pair<int, int>, std::pair<int, int>, tlb::PairHash> merges;   // (left, right) -> (rank, merged id)
    struct Added { std::string content; int id; bool special; };
    std::vector<Added> added;
    bool byte_level = false, sp_style = false, byte_fallback = false, fuse_unk = false, ignore_merges = false;
    int unk_id = -1;
    tlb::Pattern pattern = tlb::PAT_NONE;
    std::string byte_to_char[256];                    // byte-level: byte -> UTF-8 of its printable code point
    std::unordered_map<uint32_t, int> char_to_byte;   // and back
    int byte_token[256];                              // <0xHH> ids (byte fallback), -1 if absent
    std::string last_decoded;                         // storage of the string tlb_tokenizer_decode returned last
};

namespace tlb {
namespace {

const std::string kMeta = "\xE2\x96\x81";   // U+2581

void bpe_word(const tlb_tokenizer &t, std::vector<int> &sym)
{
    const int n = (int)sym.size();
    if (n < 2) return;
    std::vector<int> prev(n), next(n);
    for (int i = 0; i < n; i++) { prev[i] = i - 1; next[i] = i + 1 < n ? i + 1 : -1; }
    struct Cand { int rank, pos, left, right, merged; };
    auto cmp = [](const Cand &a, const Cand &b) { return a.rank != b.rank ? a.rank > b.rank : a.pos > b.pos; };
    std::priority_queue<Cand, std::vector<Cand>, decltype(cmp)> heap(cmp);
    auto push = [&](int i) {
        const int j = next[i];
        if (j < 0) return;
        auto it = t.merges.find({sym[i], sym[j]});
        if (it != t.merges.end()) heap.push({it->second.first, i, sym[i], sym[j], it->second.second});
    };
    for (int i = 0; i < n; i++) push(i);
    while (!heap.empty()) {
        const Cand c = heap.top();
        heap.pop();
        const int i = c.pos, j = sym[i] >= 0 ? next[i] : -1;
        if (j < 0 || sym[i] != c.left || sym[j] != c.right) continue;    // one of the halves has changed since
        sym[i] = c.merged;
        sym[j] = -1;
        next[i] = next[j];
        if (next[j] >= 0) prev[next[j]] = i;
        if (prev[i] >= 0) push(prev[i]);
        push(i);
    }
    size_t w = 0;
    for (int i = 0; i < n; i++)
        if (sym[i] >= 0) sym[w++] = sym[i];
    sym.resize(w);
}

// one piece of a pre-tokenized, byte-level text -> ids
void encode_piece_bytelevel(const tlb_tokenizer &t, const std::string &bytes, std::vector<int> &out)
{
    std::string mapped;
    for (unsigned char b : bytes) mapped += t.byte_to_char[b];
    if (t.ignore_merges) {
        auto it = t.token_to_id.find(mapped);
        if (it != t.token_to_id.end()) { out.push_back(it->second); return; }
    }
    std::vector<int> sym;
    for (unsigned char b : bytes) {
        auto it = t.token_to_id.find(t.byte_to_char[b]);
        if (it == t.token_to_id.end()) { if (t.unk_id >= 0) sym.push_back(t.unk_id); continue; }
        sym.push_back(it->second);
    }
    bpe_word(t, sym);
    out.insert(out.end(), sym.begin(), sym.end());
}

// one segment (between added tokens) -> ids
void encode_segment(const tlb_tokenizer &t, const std::string &seg, std::vector<int> &out)
{
    if (seg.empty()) return;
    if (t.byte_level) {
        std::vector<uint32_t> cps, offs;
        decode_utf8(seg, cps, offs);
        size_t i = 0;
        while (i < cps.size()) {
            size_t len = t.pattern == PAT_NONE ? cps.size() : match_at(t.pattern, cps, i);
            if (len == 0) len = 1;
            encode_piece_bytelevel(t, seg.substr(offs[i], offs[i + len] - offs[i]), out);
            i += len;
        }
        return;
    }
    // SentencePiece style: Prepend + Replace, then the merges over the code points of the whole segment
    std::string norm = t.sp_style ? kMeta : std::string();
    for (char ch : seg) {
        if (t.sp_style && ch == ' ') norm += kMeta;
        else norm += ch;
    }
    std::vector<uint32_t> cps, offs;
    decode_utf8(norm, cps, offs);
    std::vector<int> sym;
    bool last_unk = false;
    for (size_t i = 0; i < cps.size(); i++) {
        const std::string ch = norm.substr(offs[i], offs[i + 1] - offs[i]);
        auto it = t.token_to_id.find(ch);
        if (it != t.token_to_id.end()) { sym.push_back(it->second); last_unk = false; continue; }
        bool done = false;
        if (t.byte_fallback) {
            done = true;
            for (unsigned char b : ch) done = done && t.byte_token[b] >= 0;
            if (done) for (unsigned char b : ch) sym.push_back(t.byte_token[b]);
        }
        if (done) { last_unk = false; continue; }
        if (t.unk_id >= 0 && !(t.fuse_unk && last_unk)) sym.push_back(t.unk_id);
        last_unk = true;
    }
    bpe_word(t, sym);
    out.insert(out.end(), sym.begin(), sym.end());
}

// text -> ids: added tokens first (leftmost, the longest at a position), the stretches between them through the model
void encode_text(const tlb_tokenizer &t, const std::string &text, std::vector<int> &out)
{
    size_t seg0 = 0, i = 0;
    while (i < text.size()) {
        const tlb_tokenizer::Added *best = nullptr;
        for (auto &a : t.added)
            if (!a.content.empty() && text.compare(i, a.content.size(), a.content) == 0 && (!best || a.content.size() > best->content.size())) best = &a;
        if (!best) { i++; continue; }
        encode_segment(t, text.substr(seg0, i - seg0), out);
        out.push_back(best->id);
        i += best->content.size();
        seg0 = i;
    }
    encode_segment(t, text.substr(seg0), out);
}

bool is_special(const tlb_tokenizer &t, int id)
{
    for (auto &a : t.added)
        if (a.id == id && a.special) return true;
    return false;
}

// ids -> text, special tokens left out (the crate's decode(ids, skip_special_tokens = true) with the file's decoder)
std::string decode_ids(const tlb_tokenizer &t, const std::vector<int> &ids)
{
    std::string bytes;
    for (int id : ids) {
        if (id < 0 || id >= (int)t.id_to_token.size() || is_special(t, id)) continue;
        const std::string &tok = t.id_to_token[id];
        if (t.byte_level) {
            std::vector<uint32_t> cps, offs;
            decode_utf8(tok, cps, offs);
            for (size_t i = 0; i < cps.size(); i++) {
                auto it = t.char_to_byte.find(cps[i]);
                if (it != t.char_to_byte.end()) bytes += (char)it->second;
                else bytes += tok.substr(offs[i], offs[i + 1] - offs[i]);   // an added token's text: as it is
            }
        } else if (t.byte_fallback && tok.size() == 6 && tok.compare(0, 3, "<0x") == 0 && tok[5] == '>') {
            bytes += (char)strtol(tok.substr(3, 2).c_str(), nullptr, 16);
        } else {
            size_t p = 0;
            while (p < tok.size()) {
                if (t.sp_style && tok.compare(p, kMeta.size(), kMeta) == 0) { bytes += ' '; p += kMeta.size(); }
                else bytes += tok[p++];
            }
        }
    }
    // what is not UTF-8 comes out as U+FFFD, as a lossy conversion gives
    std::vector<uint32_t> cps, offs;
    decode_utf8(bytes, cps, offs);
    std::string text;
    for (uint32_t cp : cps) put_utf8(text, cp);
    if (t.sp_style && !text.empty() && text[0] == ' ') text.erase(0, 1);    // Strip(" ", 1, 0)
    return text;
}

tlb_status load_json(tlb_tokenizer *t, const JVal &root)
{
    const JVal *model = root.get("model");
    if (!model || !model->is(JVal::OBJ)) return fail(TLB_ERR_ARG, "tokenizer.json: no model");
    const JVal *type = model->get("type");
    if (type && type->is(JVal::STR) && type->str != "BPE") return fail(TLB_ERR_TYPE, "tokenizer.json: model type %s is not supported (BPE only)", type->str.c_str());
    const JVal *vocab = model->get("vocab"), *merges = model->get("merges");
    if (!vocab || !vocab->is(JVal::OBJ) || !merges || !merges->is(JVal::ARR)) return fail(TLB_ERR_ARG, "tokenizer.json: BPE model without vocab or merges");
    size_t max_id = 0;
    for (auto &kv : vocab->obj) {
        if (!kv.second.is(JVal::NUM) || kv.second.num < 0 || kv.second.num > 1e8) return fail(TLB_ERR_ARG, "tokenizer.json: bad vocabulary id");
        max_id = std::max(max_id, (size_t)kv.second.num);
    }
    const JVal *added = root.get("added_tokens");
    if (added && added->is(JVal::ARR))
        for (auto &a : added->arr) {
            const JVal *id = a.get("id"), *content = a.get("content"), *special = a.get("special");
            if (!id || !id->is(JVal::NUM) || !content || !content->is(JVal::STR) || id->num < 0 || id->num > 1e8) return fail(TLB_ERR_ARG, "tokenizer.json: bad added token");
            t->added.push_back({content->str, (int)id->num, special && special->is(JVal::BOOL) && special->b});
            max_id = std::max(max_id, (size_t)id->num);
        }
    t->id_to_token.assign(max_id + 1, std::string());
    for (auto &kv : vocab->obj) {
        t->id_to_token[(size_t)kv.second.num] = kv.first;
        t->token_to_id[kv.first] = (int)kv.second.num;
    }
    for (auto &a : t->added) {
        t->id_to_token[a.id] = a.content;
        t->token_to_id[a.content] = a.id;
    }
    int rank = 0;
    for (auto &m : merges->arr) {
        std::string l, r;
        if (m.is(JVal::ARR) && m.arr.size() == 2 && m.arr[0].is(JVal::STR) && m.arr[1].is(JVal::STR)) { l = m.arr[0].str; r = m.arr[1].str; }
        else if (m.is(JVal::STR)) {
            const size_t sp = m.str.find(' ');
            if (sp == std::string::npos) return fail(TLB_ERR_ARG, "tokenizer.json: bad merge '%s'", m.str.c_str());
            l = m.str.substr(0, sp); r = m.str.substr(sp + 1);
        } else return fail(TLB_ERR_ARG, "tokenizer.json: bad merge entry");
        auto a = t->token_to_id.find(l), b = t->token_to_id.find(r), c = t->token_to_id.find(l + r);
        if (a == t->token_to_id.end() || b == t->token_to_id.end() || c == t->token_to_id.end())
            return fail(TLB_ERR_ARG, "tokenizer.json: merge '%s' + '%s' refers to tokens outside the vocabulary", l.c_str(), r.c_str());
        t->merges.emplace(std::make_pair(a->second, b->second), std::make_pair(rank++, c->second));
    }
    auto flag = [&](const char *k) { const JVal *v = model->get(k); return v && v->is(JVal::BOOL) && v->b; };
    t->byte_fallback = flag("byte_fallback");
    t->fuse_unk = flag("fuse_unk");
    t->ignore_merges = flag("ignore_merges");
    if (const JVal *u = model->get("unk_token"))
        if (u->is(JVal::STR)) { auto it = t->token_to_id.find(u->str); if (it != t->token_to_id.end()) t->unk_id = it->second; }
    for (int b = 0; b < 256; b++) {
        char name[8];
        snprintf(name, sizeof name, "<0x%02X>", b);
        auto it = t->token_to_id.find(name);
        t->byte_token[b] = it == t->token_to_id.end() ? -1 : it->second;
    }
    // pre-tokenizer: ByteLevel (alone or in a Sequence behind a Split with a pattern the scanner knows)
    std::vector<const JVal *> pres;
    if (const JVal *pre = root.get("pre_tokenizer")) {
        if (pre->is(JVal::OBJ)) {
            const JVal *pt = pre->get("type"), *seq = pre->get("pretokenizers");
            if (pt && pt->is(JVal::STR) && pt->str == "Sequence" && seq && seq->is(JVal::ARR)) for (auto &e : seq->arr) pres.push_back(&e);
            else pres.push_back(pre);
        }
    }
    for (const JVal *e : pres) {
        const JVal *pt = e->get("type");
        if (!pt || !pt->is(JVal::STR)) continue;
        if (pt->str == "ByteLevel") {
            t->byte_level = true;
            const JVal *ur = e->get("use_regex"), *ps = e->get("add_prefix_space");
            if (ps && ps->is(JVal::BOOL) && ps->b) return fail(TLB_ERR_TYPE, "tokenizer.json: ByteLevel with add_prefix_space is not supported");
            if ((!ur || !ur->is(JVal::BOOL) || ur->b) && t->pattern == PAT_NONE) t->pattern = PAT_GPT2;   // its own built-in split
        } else if (pt->str == "Split") {
            const JVal *pat = e->get("pattern"), *rx = pat ? pat->get("Regex") : nullptr, *beh = e->get("behavior");
            if (!rx || !rx->is(JVal::STR)) return fail(TLB_ERR_TYPE, "tokenizer.json: Split without a regex is not supported");
            if (beh && beh->is(JVal::STR) && beh->str != "Isolated") return fail(TLB_ERR_TYPE, "tokenizer.json: Split behaviour %s is not supported", beh->str.c_str());
            if (rx->str == kLlama3Pattern) t->pattern = PAT_LLAMA3;
            else if (rx->str == kGpt2Pattern) t->pattern = PAT_GPT2;
            else return fail(TLB_ERR_TYPE, "tokenizer.json: the split pattern is neither Llama-3's nor GPT-2's");
        } else return fail(TLB_ERR_TYPE, "tokenizer.json: pre-tokenizer %s is not supported", pt->str.c_str());
    }
    // normalizer: none, or Prepend(U+2581) + Replace(" ", U+2581)
    if (const JVal *nz = root.get("normalizer")) {
        if (nz->is(JVal::OBJ)) {
            std::vector<const JVal *> ns;
            const JVal *nt = nz->get("type"), *seq = nz->get("normalizers");
            if (nt && nt->is(JVal::STR) && nt->str == "Sequence" && seq && seq->is(JVal::ARR)) for (auto &e : seq->arr) ns.push_back(&e);
            else ns.push_back(nz);
            bool prepend = false, replace = false;
            for (const JVal *e : ns) {
                const JVal *et = e->get("type");
                if (et && et->is(JVal::STR) && et->str == "Prepend" && e->get("prepend") && e->get("prepend")->str == kMeta) prepend = true;
                else if (et && et->is(JVal::STR) && et->str == "Replace" && e->get("content") && e->get("content")->str == kMeta) replace = true;
                else return fail(TLB_ERR_TYPE, "tokenizer.json: normalizer %s is not supported", et && et->is(JVal::STR) ? et->str.c_str() : "?");
            }
            if (!(prepend && replace)) return fail(TLB_ERR_TYPE, "tokenizer.json: only the Prepend + Replace normalizer pair is supported");
            if (t->byte_level) return fail(TLB_ERR_TYPE, "tokenizer.json: a normalizer in front of a byte-level model is not supported");
            t->sp_style = true;
        }
    }
    if (t->byte_level) {
        // the GPT-2 table: printable bytes stand for themselves, the others for U+0100 ...
        int extra = 0;
        for (int b = 0; b < 256; b++) {
            const bool keep = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
            const uint32_t cp = keep ? (uint32_t)b : 256u + (uint32_t)extra++;
            put_utf8(t->byte_to_char[b], cp);
            t->char_to_byte[cp] = b;
        }
    }
    return TLB_OK;
}

}  // namespace
}  // namespace tlb

using namespace tlb;

extern "C" {

tlb_status tlb_tokenizer_new(tlb_tokenizer **out, const char *path)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!path) return fail(TLB_ERR_NULL, "null path");
    std::ifstream f(path, std::ios::binary);
    if (!f) return fail(TLB_ERR_ARG, "Failed to load tokenizer: cannot open %s", path);
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string text = ss.str();
    JReader r{text.data(), text.data() + text.size()};
    JVal root;
    if (!r.value(root) || !root.is(JVal::OBJ)) return fail(TLB_ERR_ARG, "Failed to load tokenizer: %s is not a JSON object", path);
    tlb_tokenizer *t = new tlb_tokenizer();
    tlb_status st = load_json(t, root);
    if (st != TLB_OK) { delete t; return st; }
    *out = t;
    return TLB_OK;
}

tlb_status tlb_tokenizer_free(tlb_tokenizer *t)
{
    delete t;
    return TLB_OK;
}

int64_t tlb_tokenizer_vocab_size(const tlb_tokenizer *t) { return t ? (int64_t)t->id_to_token.size() : 0; }

const char *tlb_tokenizer_id_to_token(const tlb_tokenizer *t, int64_t id)
{
    if (!t || id < 0 || id >= (int64_t)t->id_to_token.size()) return nullptr;
    return t->id_to_token[(size_t)id].c_str();
}

tlb_status tlb_tokenizer_encode_ids(const tlb_tokenizer *t, const char *text, int32_t *ids, int64_t cap, int64_t *n)
{
    if (!t || !text || !n) return fail(TLB_ERR_NULL, "tokenizer encode: null argument");
    std::vector<int> v;
    encode_text(*t, text, v);
    *n = (int64_t)v.size();
    if (ids) {
        if ((int64_t)v.size() > cap) return fail(TLB_ERR_SHAPE, "tokenizer encode: %zu ids do not fit a buffer of %lld", v.size(), (long long)cap);
        for (size_t i = 0; i < v.size(); i++) ids[i] = v[i];
    }
    return TLB_OK;
}

static tlb_status ids_tensor(tlb_tensor **out, const std::vector<float> &ids)
{
    const int64_t shape[1] = {(int64_t)ids.size()};
    return tlb_tensor_from_host(out, ids.data(), TLB_F32, shape, 1);
}

tlb_status tlb_tokenizer_encode(tlb_tensor **out, const tlb_tokenizer *t, const char *text)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!t || !text) return fail(TLB_ERR_NULL, "tokenizer encode: null argument");
    std::vector<int> v;
    encode_text(*t, text, v);
    std::vector<float> ids(1, 1.0f);      // the runtime prepends BOS = 1 itself (tokenizer.rs:58)
    for (int id : v) ids.push_back((float)id);
    return ids_tensor(out, ids);
}

tlb_status tlb_tokenizer_encode_chat(tlb_tensor **out, const tlb_tokenizer *t, const char *user_text)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!t || !user_text) return fail(TLB_ERR_NULL, "tokenizer encode_chat: null argument");
    // the Llama-3 template with the ids of its special tokens as the runtime hard-codes them (tokenizer.rs:147-203)
    const float BOS = 128000.f, START_HDR = 128006.f, END_HDR = 128007.f, EOT = 128009.f;
    std::vector<float> ids;
    auto text = [&](const char *s) { std::vector<int> v; encode_text(*t, s, v); for (int id : v) ids.push_back((float)id); };
    auto turn = [&](const char *role, const char *body) {
        ids.push_back(START_HDR); text(role); ids.push_back(END_HDR); text("\n\n");
        if (body) { text(body); ids.push_back(EOT); }
    };
    ids.push_back(BOS);
    turn("system", "You are a helpful assistant.");
    turn("user", user_text);
    turn("assistant", nullptr);
    return ids_tensor(out, ids);
}

tlb_status tlb_tokenizer_encode_chat_zephyr(tlb_tensor **out, const tlb_tokenizer *t, const char *user_text)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!t || !user_text) return fail(TLB_ERR_NULL, "tokenizer encode_chat_zephyr: null argument");
    // one string, so that </s> is found as the added token it is; BOS = 1 in front (tokenizer.rs:210-245)
    const std::string full = std::string("<|system|>\nYou are a helpful assistant.</s>\n<|user|>\n") + user_text + "</s>\n<|assistant|>\n";
    std::vector<int> v;
    encode_text(*t, full, v);
    std::vector<float> ids(1, 1.0f);
    for (int id : v) ids.push_back((float)id);
    return ids_tensor(out, ids);
}

const char *tlb_tokenizer_decode_ids(tlb_tokenizer *t, const int32_t *ids, int64_t n)
{
    if (!t || (!ids && n > 0) || n < 0) return "";
    if (n == 1) {
        // one token: its text straight from the vocabulary, because decode() would drop a leading space (tokenizer.rs:89-117)
        const char *tok = tlb_tokenizer_id_to_token(t, ids[0]);
        std::string s = tok ? tok : "";
        if (s.size() == 6 && s.compare(0, 3, "<0x") == 0 && s[5] == '>') {
            char *e = nullptr;
            const long b = strtol(s.substr(3, 2).c_str(), &e, 16);
            if (e && *e == 0) { t->last_decoded.assign(1, (char)b); return t->last_decoded.c_str(); }
        }
        if (s.size() >= 4 && s.compare(0, 2, "<|") == 0 && s.compare(s.size() - 2, 2, "|>") == 0) s.clear();
        std::string r;
        size_t p = 0;
        while (p < s.size()) {
            if (s.compare(p, 3, kMeta) == 0) { r += ' '; p += 3; }
            else if (s.compare(p, 2, "\xC4\xA0") == 0) { r += ' '; p += 2; }     // U+0120
            else if (s.compare(p, 2, "\xC4\x8A") == 0) { r += '\n'; p += 2; }    // U+010A
            else r += s[p++];
        }
        t->last_decoded = r;
        return t->last_decoded.c_str();
    }
    std::vector<int> v(ids, ids + n);
    t->last_decoded = decode_ids(*t, v);
    return t->last_decoded.c_str();
}

const char *tlb_tokenizer_decode(tlb_tokenizer *t, const tlb_tensor *ids)
{
    if (!t || !ids || ids->dt != TLB_F32) return "";
    const int64_t n = ids->numel();
    std::vector<float> host((size_t)n);
    if (n > 0 && tlb_tensor_to_host(ids, host.data(), (size_t)n * sizeof(float)) != TLB_OK) return "";
    std::vector<int32_t> v((size_t)n);
    for (int64_t i = 0; i < n; i++) v[i] = (int32_t)(uint32_t)host[i];     // `f as u32`
    return tlb_tokenizer_decode_ids(t, v.data(), n);
}

}  // extern "C"
