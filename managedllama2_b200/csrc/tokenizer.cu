// Tokenizer of GilesBathgate/ManagedLlama2 (src/Tokenizer.cs:27-171) as host code behind the C ABI: tokenizer.bin reader,
// Encode (dummy prefix, per-character lookup with byte fallback, greedy best-score pair merging) and the stateful Decode
// (leading-space strip after BOS, <0xNN> byte pieces collected into UTF-8 characters). The reference works on UTF-16
// strings: lookups compare UTF-16 code units ordinally, Encode walks UTF-16 code units (so characters outside the basic
// plane always take the byte fallback), and its StrLookup treats a hit at index 0 of the sorted vocabulary as a miss
// (`i > 0`, :92); all three are kept. No device code in this file.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/ml2b200.h"
#include "host_common.hpp"

using namespace ml2;

namespace {

constexpr int kBOS = 1, kEOS = 2;

// UTF-8 -> UTF-16 code units; malformed input becomes U+FFFD, one per offending byte run (as a lenient decoder does)
std::u16string utf16_of(const std::string& s)
{
    std::u16string out;
    const unsigned char* p = reinterpret_cast<const unsigned char*>(s.data());
    const size_t n = s.size();
    size_t i = 0;
    while (i < n) {
        const unsigned char c = p[i];
        uint32_t cp = 0xFFFD;
        size_t len = 1;
        if (c < 0x80) {
            cp = c;
        } else if (c >= 0xC2 && c <= 0xDF && i + 1 < n && (p[i + 1] & 0xC0) == 0x80) {
            cp = ((c & 0x1Fu) << 6) | (p[i + 1] & 0x3Fu);
            len = 2;
        } else if (c >= 0xE0 && c <= 0xEF && i + 2 < n && (p[i + 1] & 0xC0) == 0x80 && (p[i + 2] & 0xC0) == 0x80) {
            const uint32_t v = ((c & 0x0Fu) << 12) | ((p[i + 1] & 0x3Fu) << 6) | (p[i + 2] & 0x3Fu);
            if (v >= 0x800 && !(v >= 0xD800 && v <= 0xDFFF)) { cp = v; len = 3; }
        } else if (c >= 0xF0 && c <= 0xF4 && i + 3 < n && (p[i + 1] & 0xC0) == 0x80 && (p[i + 2] & 0xC0) == 0x80 && (p[i + 3] & 0xC0) == 0x80) {
            const uint32_t v = ((c & 0x07u) << 18) | ((p[i + 1] & 0x3Fu) << 12) | ((p[i + 2] & 0x3Fu) << 6) | (p[i + 3] & 0x3Fu);
            if (v >= 0x10000 && v <= 0x10FFFF) { cp = v; len = 4; }
        }
        if (cp >= 0x10000) {
            cp -= 0x10000;
            out.push_back((char16_t)(0xD800 + (cp >> 10)));
            out.push_back((char16_t)(0xDC00 + (cp & 0x3FF)));
        } else {
            out.push_back((char16_t)cp);
        }
        i += len;
    }
    return out;
}

void append_utf8(std::string& out, uint32_t cp)
{
    if (cp < 0x80) {
        out.push_back((char)cp);
    } else if (cp < 0x800) {
        out.push_back((char)(0xC0 | (cp >> 6)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
        out.push_back((char)(0xE0 | (cp >> 12)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
        out.push_back((char)(0xF0 | (cp >> 18)));
        out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    }
}

// UTF-16 code units -> UTF-8; a lone surrogate becomes U+FFFD (Encoding.UTF8.GetBytes)
std::string utf8_of(const std::u16string& s)
{
    std::string out;
    for (size_t i = 0; i < s.size(); ++i) {
        uint32_t c = s[i];
        if (c >= 0xD800 && c <= 0xDBFF && i + 1 < s.size() && s[i + 1] >= 0xDC00 && s[i + 1] <= 0xDFFF) {
            c = 0x10000 + ((c - 0xD800) << 10) + (s[i + 1] - 0xDC00);
            ++i;
        } else if (c >= 0xD800 && c <= 0xDFFF) {
            c = 0xFFFD;
        }
        append_utf8(out, c);
    }
    return out;
}

bool is_white(char16_t c)   // char.IsWhiteSpace
{
    return (c >= 0x0009 && c <= 0x000D) || c == 0x0020 || c == 0x0085 || c == 0x00A0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
           c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}

struct Entry {
    std::u16string str;
    int id;
};

}  // namespace

struct ml2_tokenizer {
    std::vector<std::u16string> vocab;
    std::vector<float> scores;
    std::vector<Entry> sorted;
    int max_token_length = 0;
    std::string multibyte;   // bytes of <0xNN> pieces waiting to form characters (Decode is stateful, src/Tokenizer.cs:88)

    int lookup(const std::u16string& s) const   // StrLookup, src/Tokenizer.cs:88-93
    {
        auto it = std::lower_bound(sorted.begin(), sorted.end(), s, [](const Entry& e, const std::u16string& k) { return e.str < k; });
        if (it == sorted.end() || it->str != s) return -1;
        return (it - sorted.begin()) > 0 ? it->id : -1;   // a hit at index 0 counts as a miss there, so it does here
    }
};

extern "C" {

int ml2_tokenizer_open(const char* path, int vocab_size, ml2_tokenizer** out)
{
    if (!path || !out || vocab_size <= 0) return fail(ML2_E_INVALID, "tokenizer_open: bad argument");
    *out = nullptr;
    FILE* f = fopen(path, "rb");
    if (!f) return fail(ML2_E_INVALID, "tokenizer_open: cannot open %s", path);
    ml2_tokenizer* t = new ml2_tokenizer;
    auto bad = [&](const char* why) {
        fclose(f);
        delete t;
        return fail(ML2_E_INVALID, "tokenizer_open: %s: %s", path, why);
    };
    int32_t mtl = 0;
    if (fread(&mtl, 4, 1, f) != 1) return bad("no header");
    t->max_token_length = mtl;
    t->vocab.resize((size_t)vocab_size);
    t->scores.resize((size_t)vocab_size);
    t->sorted.resize((size_t)vocab_size);
    for (int i = 0; i < vocab_size; ++i) {   // src/Tokenizer.cs:38-48
        float score;
        int32_t len;
        if (fread(&score, 4, 1, f) != 1 || fread(&len, 4, 1, f) != 1 || len < 0 || len > (1 << 20)) return bad("truncated or malformed entry");
        std::string piece((size_t)len, '\0');
        if (len > 0 && fread(&piece[0], 1, (size_t)len, f) != (size_t)len) return bad("truncated piece");
        t->scores[(size_t)i] = score;
        t->vocab[(size_t)i] = utf16_of(piece);
        t->sorted[(size_t)i] = Entry{t->vocab[(size_t)i], i};
    }
    fclose(f);
    std::stable_sort(t->sorted.begin(), t->sorted.end(), [](const Entry& a, const Entry& b) { return a.str < b.str; });   // ordinal on UTF-16 units
    *out = t;
    return ML2_OK;
}

int ml2_tokenizer_close(ml2_tokenizer* t)
{
    delete t;
    return ML2_OK;
}

int ml2_tokenizer_encode(ml2_tokenizer* t, const char* prompt_utf8, int bos, int eos, int* out_tokens, int capacity, int* n_out)
{
    if (!t || !prompt_utf8 || !n_out || (capacity > 0 && !out_tokens)) return fail(ML2_E_INVALID, "tokenizer_encode: null argument");
    const std::u16string prompt = utf16_of(prompt_utf8);
    std::vector<int> tokens;
    tokens.reserve(prompt.size() + 3);
    if (bos) tokens.push_back(kBOS);
    if (!prompt.empty()) {   // dummy prefix, src/Tokenizer.cs:103-107
        const int dummy = t->lookup(u" ");
        if (dummy < 0) return fail(ML2_E_INVALID, "tokenizer_encode: the vocabulary has no \" \" piece (the reference would index with -1)");
        tokens.push_back(dummy);
    }
    char16_t prev = 0;
    for (const char16_t c : prompt) {   // src/Tokenizer.cs:109-130
        const int id = t->lookup(std::u16string(1, c));
        if (id != -1) {
            tokens.push_back(id);
            continue;
        }
        if (c >= 0xD800 && c <= 0xDBFF) {
            prev = c;
            continue;
        }
        std::u16string chars;
        if (prev >= 0xD800 && prev <= 0xDBFF && c >= 0xDC00 && c <= 0xDFFF) chars.push_back(prev);
        chars.push_back(c);
        for (const unsigned char b : utf8_of(chars)) tokens.push_back((int)b + 3);
        prev = 0;
    }
    // merge the best-scoring adjacent pair until none is in the vocabulary (src/Tokenizer.cs:134-166)
    std::u16string buf;
    for (;;) {
        float best_score = -3.402823466e+38f;   // float.MinValue
        int best_id = -1, best_idx = -1;
        for (size_t i = 0; i + 1 < tokens.size(); ++i) {
            const int a = tokens[i], b = tokens[i + 1];
            if (a < 0 || b < 0 || a >= (int)t->vocab.size() || b >= (int)t->vocab.size())
                return fail(ML2_E_INVALID, "tokenizer_encode: byte token %d outside the vocabulary", a >= (int)t->vocab.size() ? a : b);
            buf = t->vocab[(size_t)a];
            buf += t->vocab[(size_t)b];
            const int id = t->lookup(buf);
            if (id != -1 && t->scores[(size_t)id] > best_score) {
                best_score = t->scores[(size_t)id];
                best_id = id;
                best_idx = (int)i;
            }
        }
        if (best_idx == -1) break;
        tokens[(size_t)best_idx] = best_id;
        tokens.erase(tokens.begin() + best_idx + 1);
    }
    if (eos) tokens.push_back(kEOS);
    *n_out = (int)tokens.size();
    if ((int)tokens.size() > capacity) return fail(ML2_E_INVALID, "tokenizer_encode: %d tokens, room for %d", (int)tokens.size(), capacity);
    if (!tokens.empty()) memcpy(out_tokens, tokens.data(), tokens.size() * sizeof(int));
    return ML2_OK;
}

int ml2_tokenizer_decode(ml2_tokenizer* t, int prev, int token, char* out_utf8, int capacity, int* n_out)
{
    if (!t || !out_utf8 || !n_out || capacity <= 0) return fail(ML2_E_INVALID, "tokenizer_decode: null argument");
    if (token < 0 || token >= (int)t->vocab.size()) return fail(ML2_E_INVALID, "tokenizer_decode: token %d", token);
    std::u16string piece = t->vocab[(size_t)token];
    if (piece.empty()) return fail(ML2_E_INVALID, "tokenizer_decode: token %d has an empty piece (the reference would index past its end)", token);
    if (prev == kBOS && piece[0] == u' ') {   // src/Tokenizer.cs:60-61
        size_t k = 0;
        while (k < piece.size() && is_white(piece[k])) ++k;
        piece.erase(0, k);
    }
    // ^<0x([0-9A-F]{2})>$ (a final newline after '>' is allowed by '$')
    bool is_byte = false;
    unsigned value = 0;
    const size_t n = piece.size();
    if ((n == 6 || (n == 7 && piece[6] == u'\n')) && piece[0] == u'<' && piece[1] == u'0' && piece[2] == u'x' && piece[5] == u'>') {
        auto hex = [](char16_t c) -> int { return (c >= u'0' && c <= u'9') ? c - u'0' : ((c >= u'A' && c <= u'F') ? c - u'A' + 10 : -1); };
        const int hi = hex(piece[3]), lo = hex(piece[4]);
        if (hi >= 0 && lo >= 0) {
            is_byte = true;
            value = (unsigned)(hi * 16 + lo);
        }
    }
    std::string result;
    bool done = false;
    if (is_byte) {
        t->multibyte.push_back((char)value);
        if (value > 0x80 || (value & 0xC0) == 0x80) done = true;   // wait for the rest of the character (:72-73)
    }
    if (!done) {
        if (t->multibyte.empty()) {
            result = utf8_of(piece);
        } else {
            result = utf8_of(utf16_of(t->multibyte));   // Encoding.UTF8.GetString: malformed bytes become U+FFFD
            if (!is_byte) result += utf8_of(piece);
            t->multibyte.clear();
        }
    }
    *n_out = (int)result.size();
    if ((int)result.size() + 1 > capacity) return fail(ML2_E_INVALID, "tokenizer_decode: %d bytes, room for %d", (int)result.size() + 1, capacity);
    memcpy(out_utf8, result.c_str(), result.size() + 1);
    return ML2_OK;
}

}  // extern "C"
