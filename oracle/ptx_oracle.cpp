// CPU oracle for the PTX front end.  TEST INFRASTRUCTURE ONLY: nothing in the product may include, link or call this.
//
// A plain, sequential C++17 restatement of ZLUDA's ptx_parser (ptx_parser/src/lib.rs): a maximal-munch lexer for the
// token set of lib.rs:1930-2030 (+ one literal per opcode and modifier), a backtracking recursive-descent parser that
// follows lib.rs:503-1540 function by function and in the same alternative order, the generated instruction parser of
// ptx_parser_macros/src/lib.rs:472-911 interpreted over tables produced from the grammar spec, the error policy of
// lib.rs:392-501, and a canonical text dump of the AST (the reference AST has no Debug impl; the dump prints it
// "as if" every type derived Debug, floats as bit patterns).
//
// Parity status.  The reference cannot be built here (no Rust toolchain; logos 0.14.2 and winnow 0.6.20 are not
// vendored), so the lexer follows the published semantics of those crates: longest match, literal tokens beat
// priority-0 regexes on ties, winnow `alt`/`opt`/`repeat`/`separated` backtracking.  It is pinned against the
// reference's own fixtures and inline tests (tests/test_oracle_reference_vectors.py).  Parity unpinned: the byte span
// reported for a lex error, and the relative order of several errors raised inside one instruction.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

#include "gen/ptx_tables.h"

namespace {

using sv = std::string_view;

// =============================================================================================== lexer
struct Tok {
    uint16_t kind;
    uint32_t start, end;
};

inline bool is_alpha(unsigned char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z'); }
inline bool is_digit(unsigned char c) { return c >= '0' && c <= '9'; }
inline bool is_alnum(unsigned char c) { return is_alpha(c) || is_digit(c); }
inline bool is_identc(unsigned char c) { return is_alnum(c) || c == '_' || c == '$'; }
inline bool is_sigil(unsigned char c) { return c == '_' || c == '$' || c == '%'; }
inline bool is_ws(unsigned char c) {
    // Rust regex \s on bytes of valid UTF-8 text: ASCII whitespace (space, \t \n \v \f \r).
    return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == '\v' || c == '\f';
}

struct Keywords {
    std::unordered_map<sv, uint16_t> map;
    Keywords() {
        for (int k = 0; k < T_COUNT; k++) {
            const char* t = ptx_tok_text[k];
            if (t[0] && (k >= T_WARP_SZ)) map.emplace(sv(t), (uint16_t)k);
        }
    }
};
const Keywords& keywords() {
    static Keywords k;
    return k;
}

// literals that contain "::" (lib.rs rules with {::suffix}); each extends a DotIdent-shaped prefix
const char* const kColonLiterals[] = {
    ".L1::evict_normal", ".L1::evict_unchanged", ".L1::evict_first", ".L1::evict_last", ".L1::no_allocate",
    ".L2::cache_hint", ".L2::64B", ".L2::128B", ".L2::256B", ".L2::evict_last", ".L2::evict_normal",
    ".L2::evict_first", ".L2::evict_unchanged", ".param::entry", ".param::func", ".shared::cta", ".shared::cluster"};

// Longest match at `p` (p < n, text[p] is not whitespace and not the start of a comment).
// Returns the token kind and sets *len; kind T_ERROR means no rule matches (len = bytes to skip).
uint16_t lex_one(const char* s, size_t p, size_t n, size_t* len) {
    unsigned char c = s[p];
    auto at = [&](size_t i) -> unsigned char { return i < n ? (unsigned char)s[i] : 0; };
    switch (c) {
    case ',': *len = 1; return T_COMMA;
    case ':': *len = 1; return T_COLON;
    case ';': *len = 1; return T_SEMI;
    case '@': *len = 1; return T_AT;
    case '|': *len = 1; return T_PIPE;
    case '!': *len = 1; return T_EXCL;
    case '(': *len = 1; return T_LPAREN;
    case ')': *len = 1; return T_RPAREN;
    case '[': *len = 1; return T_LBRACKET;
    case ']': *len = 1; return T_RBRACKET;
    case '{': *len = 1; return T_LBRACE;
    case '}': *len = 1; return T_RBRACE;
    case '<': *len = 1; return T_LT;
    case '>': *len = 1; return T_GT;
    case '-': *len = 1; return T_MINUS;
    case '+': *len = 1; return T_PLUS;
    case '=': *len = 1; return T_EQ;
    case '"': {
        size_t q = p + 1;
        while (q < n && s[q] != '"') q++;
        if (q >= n) { *len = n - p; return T_ERROR; }   // unterminated string
        *len = q + 1 - p;
        return T_STRING;
    }
    default: break;
    }
    if (is_alpha(c) || is_sigil(c)) {
        size_t q = p + 1;
        while (q < n && is_identc(s[q])) q++;
        if (is_sigil(c) && q == p + 1) { *len = 1; return T_ERROR; }   // [_$%] needs one more identifier character
        *len = q - p;
        if (is_alpha(c)) {
            auto it = keywords().map.find(sv(s + p, q - p));
            if (it != keywords().map.end()) return it->second;
        }
        return T_IDENT;
    }
    if (c == '.') {
        unsigned char d = at(p + 1);
        if (is_alpha(d) || is_sigil(d)) {
            size_t q = p + 2;
            while (q < n && is_identc(s[q])) q++;
            if (is_sigil(d) && q == p + 2) { *len = 1; return T_DOT; }
            // "::" literals are longer than the DotIdent match and therefore win
            if (at(q) == ':' && at(q + 1) == ':') {
                for (const char* lit : kColonLiterals) {
                    size_t l = strlen(lit);
                    if (p + l <= n && memcmp(s + p, lit, l) == 0) {
                        *len = l;
                        return keywords().map.at(sv(lit));
                    }
                }
            }
            *len = q - p;
            auto it = keywords().map.find(sv(s + p, q - p));
            if (it != keywords().map.end()) return it->second;
            return T_DOTIDENT;
        }
        if (is_digit(d)) {
            // ".1d" ".2d" ".3d" (tex dimensions) are 3-byte literals and beat the 2-byte F64 match ".1"
            if ((d == '1' || d == '2' || d == '3') && at(p + 2) == 'd') {
                *len = 3;
                return keywords().map.at(sv(s + p, 3));
            }
            size_t q = p + 1;
            while (q < n && is_digit(s[q])) q++;
            if (at(q) == 'e' || at(q) == 'E') {
                size_t r = q + 1;
                if (at(r) == '-' || at(r) == '+') r++;
                if (is_digit(at(r))) {
                    while (r < n && is_digit(s[r])) r++;
                    q = r;
                }
            }
            *len = q - p;
            return T_F64;
        }
        *len = 1;
        return T_DOT;
    }
    if (is_digit(c)) {
        if (c == '0') {
            unsigned char d = at(p + 1);
            if (d == 'x' || d == 'X') {
                size_t q = p + 2;
                while (q < n && is_alnum(s[q])) q++;
                if (q > p + 2) { *len = q - p; return T_HEX; }
            } else if (d == 'f' || d == 'F' || d == 'd' || d == 'D') {
                size_t need = (d == 'f' || d == 'F') ? 8 : 16;
                size_t q = p + 2;
                while (q < n && q < p + 2 + need && is_alnum(s[q])) q++;
                if (q == p + 2 + need) { *len = q - p; return (d == 'f' || d == 'F') ? T_F32HEX : T_F64HEX; }
            }
        }
        size_t q = p + 1;
        while (q < n && is_digit(s[q])) q++;
        // digits '.' digits+ [exponent] is an F64 and is longer than the Decimal match
        if (at(q) == '.' && is_digit(at(q + 1))) {
            size_t r = q + 1;
            while (r < n && is_digit(s[r])) r++;
            if (at(r) == 'e' || at(r) == 'E') {
                size_t e = r + 1;
                if (at(e) == '-' || at(e) == '+') e++;
                if (is_digit(at(e))) {
                    while (e < n && is_digit(s[e])) e++;
                    r = e;
                }
            }
            *len = r - p;
            return T_F64;
        }
        if (at(q) == 'U') q++;
        *len = q - p;
        return T_DECIMAL;
    }
    *len = 1;
    return T_ERROR;
}

struct LexResult {
    std::vector<Tok> toks;
    std::vector<Tok> errors;   // spans that match no rule
};

LexResult lex(const char* s, size_t n) {
    LexResult r;
    size_t p = 0;
    while (p < n) {
        unsigned char c = s[p];
        if (is_ws(c)) { p++; continue; }
        if (c == '/') {
            if (p + 1 < n && s[p + 1] == '/') {
                p += 2;
                while (p < n && s[p] != '\n' && s[p] != '\r') p++;
                continue;
            }
            if (p + 1 < n && s[p + 1] == '*') {
                size_t q = p + 2;
                bool closed = false;
                while (q + 1 < n) {
                    if (s[q] == '*' && s[q + 1] == '/') { closed = true; break; }
                    q++;
                }
                if (closed) { p = q + 2; continue; }
                // unterminated comment: reported at the end of the input (the span of a lex error is unpinned)
                r.errors.push_back({T_ERROR, (uint32_t)n, (uint32_t)n});
                p = n;
                continue;
            }
            r.errors.push_back({T_ERROR, (uint32_t)p, (uint32_t)(p + 1)});
            p++;
            continue;
        }
        size_t len = 0;
        uint16_t k = lex_one(s, p, n, &len);
        if (k == T_ERROR) r.errors.push_back({T_ERROR, (uint32_t)p, (uint32_t)(p + len)});
        else r.toks.push_back({k, (uint32_t)p, (uint32_t)(p + len)});
        p += len;
    }
    return r;
}

// =============================================================================================== AST
struct Imm {
    int kind = 0;   // 0 U64, 1 S64, 2 F32, 3 F64
    uint64_t bits = 0;
};
struct RegOrImm {
    bool is_reg = false;
    sv reg;
    Imm imm;
};
struct Operand {
    int kind = 0;   // 0 Reg, 1 RegOffset, 2 Imm, 3 VecMember, 4 VecPack
    sv name;
    int32_t offset = 0;
    uint8_t index = 0;
    Imm imm;
    std::vector<RegOrImm> pack;
    uint32_t span_start = 0, span_end = 0;
};
struct Type {
    int kind = 0;   // 0 Scalar, 1 Vector, 2 Array, 3 Texref
    int vec = 0;    // 0 = none
    int scalar = 0;
    std::vector<uint32_t> dims;
};
struct VarInfo {
    bool has_align = false;
    uint32_t align = 0;
    Type type;
    int space = 0;
    std::vector<RegOrImm> init;
};
struct Variable {
    VarInfo info;
    sv name;
};
struct MultiVar {
    bool parameterized = false;
    VarInfo info;
    std::vector<sv> names;
    uint32_t count = 0;
};
struct TypeSpace {
    Type type;
    int space;
};
struct Instruction {
    int variant = -1;
    std::vector<uint32_t> data;
    std::vector<int> args;   // operand index, or -1 for an absent optional operand
    std::vector<Operand> ops;
    sv bra_target;
    // call
    bool call_uniform = false;
    std::vector<TypeSpace> call_ret_types, call_in_types;
    std::vector<sv> call_rets;
    sv call_func;
    std::vector<int> call_inputs;
};
struct Statement {
    int kind = 0;   // 0 Label, 1 Variable, 2 Instruction, 3 Block
    sv label;
    MultiVar var;
    bool has_pred = false, pred_not = false;
    sv pred;
    Instruction ins;
    std::vector<Statement> block;
};
struct Tuning {
    int kind = 0;   // 0 MaxNReg 1 MaxNtid 2 ReqNtid 3 MinNCtaPerSm 4 NoReturn
    uint32_t v[3] = {0, 0, 0};
};
struct Function {
    std::vector<Variable> rets, inputs;
    bool is_kernel = false;
    sv name;
    std::vector<Tuning> tuning;
    bool has_body = false;
    std::vector<Statement> body;
};
struct Directive {
    bool is_method = false;
    int linking = 0;
    Variable var;
    Function func;
};
struct Module {
    uint8_t major = 0, minor = 0;
    uint32_t sm = 0;
    uint8_t address_size = 32;
    std::vector<Directive> directives;
    uint64_t invalid = 0;
};
struct Error {
    int kind, sub;
    uint32_t a, b;   // span (offset, length) or message id / auxiliary values
};

// =============================================================================================== parser
static unsigned char g_pattern_hits[PTX_N_PATTERNS];   // not thread-safe by design: read by single-threaded tests only

struct Parser {
    const char* text;
    size_t text_len;
    const std::vector<Tok>& t;
    size_t pos = 0;
    std::vector<Error>& errors;
    std::unordered_map<sv, std::pair<std::vector<TypeSpace>, std::vector<TypeSpace>>> fns;

    Parser(const char* s, size_t n, const std::vector<Tok>& toks, std::vector<Error>& e)
        : text(s), text_len(n), t(toks), errors(e) {}

    bool eof() const { return pos >= t.size(); }
    uint16_t kind() const { return pos < t.size() ? t[pos].kind : (uint16_t)0xFFFE; }
    sv tok_text(size_t i) const { return sv(text + t[i].start, t[i].end - t[i].start); }
    bool eat(uint16_t k) {
        if (kind() == k) { pos++; return true; }
        return false;
    }
    void push(int kind_, int sub = 0, uint32_t a = 0, uint32_t b = 0) { errors.push_back({kind_, sub, a, b}); }

    static bool is_opcode(uint16_t k) { return k >= T_OP_FIRST && k < T_MOD_FIRST; }
    static bool is_modifier(uint16_t k) { return k >= T_MOD_FIRST && k < T_COUNT; }

    // ---- lib.rs:155-220
    bool ident(sv* out) {
        if (eof()) return false;
        uint16_t k = kind();
        if (k == T_IDENT) {
            sv s = tok_text(pos);
            if (s.size() >= 8 && s.size() <= 9 && s.substr(0, 7) == "%envreg") {
                int v = 0;
                bool ok = true;
                for (size_t i = 7; i < s.size(); i++) {
                    if (!is_digit(s[i])) ok = false;
                    v = v * 10 + (s[i] - '0');
                }
                if (ok && s[7] != '0' && v >= 1 && v <= 32) push(E_UNSUPPORTED_SREG, 0, t[pos].start, t[pos].end - t[pos].start);
            }
            *out = s;
            pos++;
            return true;
        }
        if (is_opcode(k)) {
            *out = tok_text(pos);
            pos++;
            return true;
        }
        return false;
    }
    bool dot_ident(sv* out) {
        if (kind() == T_DOTIDENT) { *out = tok_text(pos); pos++; return true; }
        return false;
    }
    bool ident_literal(sv lit) {
        if (kind() == T_IDENT && tok_text(pos) == lit) { pos++; return true; }
        return false;
    }

    // ---- lib.rs:222-247
    bool num(sv* digits, int* radix, bool* is_unsigned) {
        if (kind() == T_HEX) {
            sv s = tok_text(pos);
            if (s.back() == 'U') { *digits = s.substr(2, s.size() - 3); *is_unsigned = true; }
            else { *digits = s.substr(2); *is_unsigned = false; }
            *radix = 16;
            pos++;
            return true;
        }
        if (kind() == T_DECIMAL) {
            sv s = tok_text(pos);
            *radix = s[0] == '0' ? 8 : 10;
            if (s.back() == 'U') { *digits = s.substr(0, s.size() - 1); *is_unsigned = true; }
            else { *digits = s; *is_unsigned = false; }
            pos++;
            return true;
        }
        return false;
    }

    // Rust {integer}::from_str_radix for a magnitude limited to `max` (positive) or `neg_max` (negative).
    // Returns -1 on success, else the IntErrorKind.
    static int parse_radix(sv s, int radix, bool negative, uint64_t limit, uint64_t* out) {
        if (s.empty()) return negative ? PI_INVALID_DIGIT : PI_EMPTY;   // "-" alone is InvalidDigit
        uint64_t v = 0;
        for (char ch : s) {
            int d;
            if (ch >= '0' && ch <= '9') d = ch - '0';
            else if (ch >= 'a' && ch <= 'z') d = ch - 'a' + 10;
            else if (ch >= 'A' && ch <= 'Z') d = ch - 'A' + 10;
            else return PI_INVALID_DIGIT;
            if (d >= radix) return PI_INVALID_DIGIT;
            if (v > (limit - (uint64_t)d) / (uint64_t)radix) return negative ? PI_NEG_OVERFLOW : PI_POS_OVERFLOW;
            v = v * radix + d;
        }
        *out = v;
        return -1;
    }

    // ---- lib.rs:263-288
    bool int_immediate(Imm* out) {
        size_t save = pos;
        bool neg = eat(T_MINUS);
        sv d; int radix; bool uns;
        if (!num(&d, &radix, &uns)) { pos = save; return false; }
        uint64_t v = 0;
        if (neg) {
            int e = parse_radix(d, radix, true, (uint64_t)1 << 63, &v);
            if (e >= 0) { push(E_PARSE_INT, e); *out = {1, 0}; }
            else *out = {1, (uint64_t)(0 - v)};
        } else if (uns) {
            int e = parse_radix(d, radix, false, UINT64_MAX, &v);
            if (e >= 0) { push(E_PARSE_INT, e); *out = {0, 0}; }
            else *out = {0, v};
        } else {
            int e = parse_radix(d, radix, false, (uint64_t)INT64_MAX, &v);
            if (e < 0) *out = {1, v};
            else {
                e = parse_radix(d, radix, false, UINT64_MAX, &v);
                if (e >= 0) { push(E_PARSE_INT, e); *out = {0, 0}; }
                else *out = {0, v};
            }
        }
        return true;
    }
    // ---- lib.rs:290-314
    bool f32_tok(Imm* out) {
        if (kind() != T_F32HEX) return false;
        uint64_t v = 0;
        int e = parse_radix(tok_text(pos).substr(2), 16, false, UINT32_MAX, &v);
        if (e >= 0) { push(E_PARSE_INT, e); v = 0; }
        *out = {2, v};
        pos++;
        return true;
    }
    bool f64_tok(Imm* out) {
        if (kind() == T_F64HEX) {
            uint64_t v = 0;
            int e = parse_radix(tok_text(pos).substr(2), 16, false, UINT64_MAX, &v);
            if (e >= 0) { push(E_PARSE_INT, e); v = 0; }
            *out = {3, v};
            pos++;
            return true;
        }
        if (kind() == T_F64) {
            std::string s(tok_text(pos));
            double d = strtod(s.c_str(), nullptr);   // correctly rounded, like Rust's str::parse::<f64>
            uint64_t v;
            memcpy(&v, &d, 8);
            *out = {3, v};
            pos++;
            return true;
        }
        return false;
    }
    // ---- lib.rs:316-350
    bool s32(int32_t* out) {
        size_t save = pos;
        bool neg = eat(T_MINUS);
        sv d; int radix; bool uns;
        if (!num(&d, &radix, &uns)) { pos = save; return false; }
        uint64_t v = 0;
        int e = parse_radix(d, radix, false, (uint64_t)INT32_MAX, &v);
        if (e >= 0) { push(E_PARSE_INT, e); *out = 0; }
        else *out = neg ? -(int32_t)v : (int32_t)v;
        return true;
    }
    bool uint_limited(uint64_t limit, uint32_t* out) {
        sv d; int radix; bool uns;
        if (!num(&d, &radix, &uns)) return false;
        uint64_t v = 0;
        int e = parse_radix(d, radix, false, limit, &v);
        if (e >= 0) { push(E_PARSE_INT, e); v = 0; }
        *out = (uint32_t)v;
        return true;
    }
    bool u32(uint32_t* out) { return uint_limited(UINT32_MAX, out); }
    bool u8(uint32_t* out) { return uint_limited(255, out); }
    // ---- lib.rs:352-390
    bool immediate_value(Imm* out) {
        if (int_immediate(out)) return true;
        if (f32_tok(out)) return true;
        if (f64_tok(out)) return true;
        if (kind() == T_WARP_SZ) { *out = {0, 32}; pos++; return true; }
        return false;
    }
    bool reg_or_immediate(RegOrImm* out) {
        Imm imm;
        if (immediate_value(&imm)) { out->is_reg = false; out->imm = imm; return true; }
        sv id;
        if (ident(&id)) { out->is_reg = true; out->reg = id; return true; }
        return false;
    }

    // ---- lib.rs:1487-1540
    bool operand(Operand* out) {
        size_t save = pos;
        *out = Operand();
        out->span_start = eof() ? 0 : t[pos].start;
        bool ok = operand_inner(out);
        if (!ok) { pos = save; return false; }
        out->span_end = t[pos - 1].end;
        return true;
    }
    bool operand_inner(Operand* out) {
        size_t save = pos;
        sv id;
        if (ident(&id)) {
            out->name = id;
            size_t after = pos;
            if (eat(T_PLUS)) {
                int32_t off;
                if (s32(&off)) { out->kind = 1; out->offset = off; return true; }
                pos = after;
            }
            sv suffix;
            if (dot_ident(&suffix)) {
                out->kind = 3;
                int idx = -1;
                if (suffix == ".x" || suffix == ".r") idx = 0;
                else if (suffix == ".y" || suffix == ".g") idx = 1;
                else if (suffix == ".z" || suffix == ".b") idx = 2;
                else if (suffix == ".w" || suffix == ".a") idx = 3;
                if (idx < 0) { push(E_WRONG_VECTOR_ELEMENT); idx = 0; }
                out->index = (uint8_t)idx;
                return true;
            }
            out->kind = 0;
            return true;
        }
        pos = save;
        Imm imm;
        if (immediate_value(&imm)) { out->kind = 2; out->imm = imm; return true; }
        pos = save;
        if (eat(T_LBRACE)) {
            std::vector<RegOrImm> pack;
            RegOrImm r;
            if (reg_or_immediate(&r)) {
                pack.push_back(r);
                while (pack.size() < 8) {
                    size_t s2 = pos;
                    if (!eat(T_COMMA)) break;
                    if (!reg_or_immediate(&r)) { pos = s2; break; }
                    pack.push_back(r);
                }
                if (eat(T_RBRACE)) { out->kind = 4; out->pack = std::move(pack); return true; }
            }
        }
        pos = save;
        return false;
    }

    // ---- variables, lib.rs:1012-1369
    int scalar_type() {
        int r = -1;
        switch (kind()) {
        case T_MOD_s8: r = ScalarType_S8; break;
        case T_MOD_s16: r = ScalarType_S16; break;
        case T_MOD_s16x2: r = ScalarType_S16x2; break;
        case T_MOD_s32: r = ScalarType_S32; break;
        case T_MOD_s64: r = ScalarType_S64; break;
        case T_MOD_u8: r = ScalarType_U8; break;
        case T_MOD_u16: r = ScalarType_U16; break;
        case T_MOD_u16x2: r = ScalarType_U16x2; break;
        case T_MOD_u32: r = ScalarType_U32; break;
        case T_MOD_u64: r = ScalarType_U64; break;
        case T_MOD_b8: r = ScalarType_B8; break;
        case T_MOD_b16: r = ScalarType_B16; break;
        case T_MOD_b32: r = ScalarType_B32; break;
        case T_MOD_b64: r = ScalarType_B64; break;
        case T_MOD_b128: r = ScalarType_B128; break;
        case T_MOD_pred: r = ScalarType_Pred; break;
        case T_MOD_f16: r = ScalarType_F16; break;
        case T_MOD_f16x2: r = ScalarType_F16x2; break;
        case T_MOD_f32: r = ScalarType_F32; break;
        case T_MOD_f64: r = ScalarType_F64; break;
        case T_MOD_bf16: r = ScalarType_BF16; break;
        case T_MOD_bf16x2: r = ScalarType_BF16x2; break;
        default: return -1;
        }
        pos++;
        return r;
    }
    int vector_prefix() {
        if (eat(T_MOD_v2)) return 2;
        if (eat(T_MOD_v4)) return 4;
        if (eat(T_MOD_v8)) return 8;
        return 0;
    }
    // opt(align.verify(power of two))
    void opt_align(bool* has, uint32_t* v) {
        size_t save = pos;
        *has = false;
        if (eat(T_DOT_ALIGN)) {
            uint32_t a;
            if (u32(&a) && __builtin_popcount(a) == 1) { *has = true; *v = a; return; }
        }
        pos = save;
    }
    bool variable_info_non_texref(bool* has_align, uint32_t* align, int* vec, int* scalar) {
        size_t save = pos;
        opt_align(has_align, align);
        *vec = vector_prefix();
        *scalar = scalar_type();
        if (*scalar < 0) { pos = save; return false; }
        return true;
    }
    bool array_dimensions(std::vector<uint32_t>* dims) {
        size_t save = pos;
        if (!eat(T_LBRACKET)) return false;
        uint32_t d = 0;
        size_t s2 = pos;
        bool has = u32(&d);
        if (!has) pos = s2;
        if (has && d == 0) { pos = save; return false; }
        if (!eat(T_RBRACKET)) { pos = save; return false; }
        dims->clear();
        dims->push_back(has ? d : 0);
        for (;;) {
            size_t s3 = pos;
            uint32_t x;
            if (eat(T_LBRACKET) && u32(&x) && x != 0 && eat(T_RBRACKET)) dims->push_back(x);
            else { pos = s3; break; }
        }
        return true;
    }
    static Imm default_imm(int scalar) {
        int k = scalar_kind(scalar);
        if (k == KIND_SIGNED) return {1, 0};
        if (k == KIND_FLOAT) return {3, 0};
        return {0, 0};
    }
    static Type maybe_array(int vec, int scalar, const std::vector<uint32_t>* dims) {
        Type ty;
        ty.vec = vec;
        ty.scalar = scalar;
        if (dims) { ty.kind = 2; ty.dims = *dims; }
        else ty.kind = vec ? 1 : 0;
        return ty;
    }
    bool multi_variable(bool extern_, int space, MultiVar* out) {
        size_t save = pos;
        bool texref = false;
        bool has_align = false;
        uint32_t align = 0;
        int vec = 0, scalar = 0;
        if (space == StateSpace_Global && (kind() == T_DOT_TEXREF || kind() == T_DOT_SURFREF)) {
            pos++;
            texref = true;
        } else if (!variable_info_non_texref(&has_align, &align, &vec, &scalar)) {
            pos = save;
            return false;
        }
        std::vector<sv> names;
        sv id;
        if (!ident(&id)) { pos = save; return false; }
        names.push_back(id);
        for (;;) {
            size_t s2 = pos;
            if (!eat(T_COMMA)) break;
            if (!ident(&id)) { pos = s2; break; }
            names.push_back(id);
        }
        bool has_count = false;
        uint32_t count = 0;
        {
            size_t s2 = pos;
            if (eat(T_LT) && u32(&count) && count != 0 && eat(T_GT)) has_count = true;
            else pos = s2;
        }
        *out = MultiVar();
        out->info.space = space;
        if (texref) {
            if (has_count) { pos = save; return false; }
            out->info.type.kind = 3;
            out->names = names;
            return true;
        }
        out->info.has_align = has_align;
        out->info.align = align;
        if (has_count) {
            if (names.size() > 1) { pos = save; return false; }
            out->parameterized = true;
            out->info.type = maybe_array(vec, scalar, nullptr);
            out->names = names;
            out->count = count;
            return true;
        }
        std::vector<uint32_t> dims;
        bool has_dims = false;
        if (space != StateSpace_Reg) has_dims = array_dimensions(&dims);
        if (space == StateSpace_Global || space == StateSpace_Const) {
            std::vector<RegOrImm> init;
            bool got = false;
            size_t s2 = pos;
            if (eat(T_EQ)) {
                if (has_dims) {
                    if (!(vec != 0 || dims[0] == 0 || dims.size() > 1) && eat(T_LBRACE)) {
                        RegOrImm r;
                        size_t s3 = pos;
                        if (dims[0] >= 1 && reg_or_immediate(&r)) {
                            init.push_back(r);
                            while (init.size() < dims[0]) {
                                size_t s4 = pos;
                                if (!eat(T_COMMA)) break;
                                if (!reg_or_immediate(&r)) { pos = s4; break; }
                                init.push_back(r);
                            }
                        } else {
                            pos = s3;
                        }
                        if (eat(T_RBRACE)) got = true;
                    }
                } else {
                    RegOrImm r;
                    if (vec == 0 && reg_or_immediate(&r)) { init.push_back(r); got = true; }
                }
            }
            if (!got) { pos = s2; init.clear(); }
            if (has_dims) {
                RegOrImm z;
                z.imm = default_imm(scalar);
                while (init.size() < dims[0]) init.push_back(z);
            } else if (!got) {
                RegOrImm z;
                z.imm = default_imm(scalar);
                init.push_back(z);
            }
            out->info.init = std::move(init);
        }
        if (has_dims && !extern_ && dims[0] == 0) { pos = save; return false; }
        out->info.type = maybe_array(vec, scalar, has_dims ? &dims : nullptr);
        out->names = names;
        return true;
    }
    // ---- lib.rs:961-1010
    bool method_parameter(int space, Variable* out) {
        size_t save = pos;
        bool has_align = false;
        uint32_t align = 0;
        int vec = 0, scalar = 0;
        sv name;
        bool ok = false;
        if (variable_info_non_texref(&has_align, &align, &vec, &scalar) && ident(&name)) ok = true;
        if (!ok) {
            pos = save;
            has_align = false;
            vec = vector_prefix();
            scalar = scalar_type();
            if (scalar >= 0) {
                if (eat(T_DOT_PTR)) eat(T_MOD_global);
                opt_align(&has_align, &align);
                if (ident(&name)) ok = true;
            }
        }
        if (!ok) { pos = save; return false; }
        std::vector<uint32_t> dims;
        bool has_dims = false;
        if (space != StateSpace_Reg) has_dims = array_dimensions(&dims);
        if (has_dims && dims[0] == 0) { pos = save; return false; }
        out->info = VarInfo();
        out->info.has_align = has_align;
        out->info.align = align;
        out->info.type = maybe_array(vec, scalar, has_dims ? &dims : nullptr);
        out->info.space = space;
        out->name = name;
        return true;
    }
    bool param_list(bool kernel, std::vector<Variable>* out) {
        size_t save = pos;
        if (!eat(T_LPAREN)) return false;
        out->clear();
        auto one = [&](Variable* v) -> bool {
            size_t s2 = pos;
            if (eat(T_MOD_param)) { if (method_parameter(StateSpace_Param, v)) return true; }
            else if (!kernel && eat(T_DOT_REG)) { if (method_parameter(StateSpace_Reg, v)) return true; }
            pos = s2;
            return false;
        };
        Variable v;
        if (one(&v)) {
            out->push_back(v);
            for (;;) {
                size_t s2 = pos;
                if (!eat(T_COMMA)) break;
                if (!one(&v)) { pos = s2; break; }
                out->push_back(v);
            }
        }
        if (!eat(T_RPAREN)) { pos = save; return false; }
        return true;
    }

    // ---- instructions: ptx_parser_macros/src/lib.rs:585-911, lib.rs:1695-1818
    struct Builder {
        Parser& p;
        Instruction& ins;
        void put(uint32_t w) { ins.data.push_back(w); }
        void arg(int i) { ins.args.push_back(i); }
        void arg_imm_u64(uint64_t v) {
            Operand o;
            o.kind = 2;
            o.imm = {0, v};
            ins.ops.push_back(o);
            ins.args.push_back((int)ins.ops.size() - 1);
        }
        void err(int kind, int sub, uint32_t a, uint32_t b) { p.push(kind, sub, a, b); }
        void err_todo(int id) { p.push(E_TODO, id); }
        bool op_as_u64(int i, uint64_t* v) {
            if (i < 0 || ins.ops[i].kind != 2 || ins.ops[i].imm.kind > 1) return false;
            *v = ins.ops[i].imm.bits;
            return true;
        }
        bool op_as_f64(int i, double* v) {
            if (i < 0 || ins.ops[i].kind != 2 || ins.ops[i].imm.kind != 3) return false;
            memcpy(v, &ins.ops[i].imm.bits, 8);
            return true;
        }
        void op_span(int i, uint32_t* off, uint32_t* len) {
            *off = ins.ops[i].span_start;
            *len = ins.ops[i].span_end - ins.ops[i].span_start;
        }
    };

    bool parse_args(const PtxPattern& pt, int i, Instruction& ins, int* av, int* aneg, int* auni) {
        if (i == pt.n_args) return true;
        uint8_t fl = ptx_pattern_args[pt.first_arg + i];
        auto inner = [&]() -> bool {
            if (!(i == 0 || (fl & PTX_ARG_PRE_PIPE))) if (!eat(T_COMMA)) return false;
            if (fl & PTX_ARG_PRE_BRACKET) if (!eat(T_LBRACKET)) return false;
            if (fl & PTX_ARG_PRE_PIPE) if (!eat(T_PIPE)) return false;
            aneg[i] = 0;
            if (fl & PTX_ARG_NEGATED) aneg[i] = eat(T_EXCL) ? 1 : 0;
            Operand op;
            if (!operand(&op)) return false;
            ins.ops.push_back(std::move(op));
            av[i] = (int)ins.ops.size() - 1;
            if (fl & PTX_ARG_POST_BRACKET) if (!eat(T_RBRACKET)) return false;
            auni[i] = 0;
            if (fl & PTX_ARG_UNIFIED) auni[i] = eat(T_MOD_unified) ? 1 : 0;
            return true;
        };
        if (!(fl & PTX_ARG_OPTIONAL)) return inner() && parse_args(pt, i + 1, ins, av, aneg, auni);
        size_t save = pos;
        if (inner() && parse_args(pt, i + 1, ins, av, aneg, auni)) return true;
        pos = save;
        av[i] = -1;
        aneg[i] = auni[i] = 0;
        return parse_args(pt, i + 1, ins, av, aneg, auni);
    }

    bool parse_pattern(int pattern, size_t mod_begin, size_t mod_end, Instruction& ins) {
        const PtxPattern& pt = ptx_patterns[pattern];
        int mv[PTX_MAX_SLOTS];
        int nslots = pt.n_unordered + pt.n_ordered;
        for (int i = 0; i < nslots; i++) mv[i] = ptx_slots[pt.first_slot + i].typed ? -1 : 0;
        auto match_slot = [&](const PtxSlot& sl, uint16_t k) -> int {   // value or -2
            for (int a = 0; a < sl.n_alt; a++)
                if (T_MOD_FIRST + ptx_alts[sl.first_alt + a].mod == k) return ptx_alts[sl.first_alt + a].value;
            return -2;
        };
        size_t end = mod_end;
        // ordered modifiers, parsed from the tail of the run
        for (int i = nslots - 1; i >= pt.n_unordered; i--) {
            const PtxSlot& sl = ptx_slots[pt.first_slot + i];
            int v = end > mod_begin ? match_slot(sl, t[end - 1].kind) : -2;
            if (v != -2) { mv[i] = v; end--; }
            else if (!sl.optional) return false;
        }
        // the rest in any order, each at most once
        bool seen[PTX_MAX_SLOTS] = {false};
        for (size_t j = mod_begin; j < end; j++) {
            bool found = false;
            for (int i = 0; i < pt.n_unordered; i++) {
                int v = match_slot(ptx_slots[pt.first_slot + i], t[j].kind);
                if (v == -2) continue;
                if (seen[i]) return false;
                seen[i] = true;
                mv[i] = v;
                found = true;
                break;
            }
            if (!found) return false;
        }
        for (int i = 0; i < pt.n_unordered; i++)
            if (!ptx_slots[pt.first_slot + i].optional && !seen[i]) return false;
        int av[PTX_MAX_ARGS], aneg[PTX_MAX_ARGS], auni[PTX_MAX_ARGS];
        for (int i = 0; i < PTX_MAX_ARGS; i++) { av[i] = -1; aneg[i] = auni[i] = 0; }
        if (!parse_args(pt, 0, ins, av, aneg, auni)) return false;
        ins.variant = pt.instr;
        Builder b{*this, ins};
        ptx_build(pattern, b, mv, av, aneg, auni);
        g_pattern_hits[pattern] = 1;      // test coverage: which patterns the inputs so far have exercised
        return true;
    }

    bool parse_instruction(Instruction* out) {
        if (eof()) return false;
        uint16_t k = kind();
        if (!is_opcode(k)) return false;
        pos++;
        Instruction& ins = *out;
        ins = Instruction();
        const PtxOpcode& op = ptx_opcodes[k - T_OP_FIRST];
        if (op.special == 1) {   // bra
            eat(T_MOD_uni);
            if (kind() != T_IDENT) return false;
            ins.variant = I_Bra;
            ins.bra_target = tok_text(pos);
            pos++;
            return true;
        }
        if (op.special == 2) return parse_call(ins);
        if (op.special == 3) {   // vshr.u32.u32.u32.mode.add d, a, b, c
            if (!(eat(T_MOD_u32) && eat(T_MOD_u32) && eat(T_MOD_u32))) return false;
            int mode;
            if (eat(T_MOD_clamp)) mode = FunnelShiftMode_Clamp;
            else if (eat(T_MOD_wrap)) mode = FunnelShiftMode_Wrap;
            else return false;
            if (!eat(T_MOD_add)) return false;
            for (int i = 0; i < 4; i++) {
                if (i && !eat(T_COMMA)) return false;
                Operand o;
                if (!operand(&o)) return false;
                ins.ops.push_back(std::move(o));
                ins.args.push_back(i);
            }
            ins.variant = I_Vshr;
            ins.data = {(uint32_t)mode, (uint32_t)VshOp_Add};
            return true;
        }
        size_t mb = pos;
        while (!eof() && is_modifier(kind())) pos++;
        size_t me = pos;
        uint64_t mask[PTX_MOD_WORDS] = {0, 0, 0};
        for (size_t j = mb; j < me; j++) {
            int m = t[j].kind - T_MOD_FIRST;
            mask[m / 64] |= 1ull << (m % 64);
        }
        for (int c = 0; c < op.n_chain; c++) {
            const PtxChain& ch = ptx_chains[op.first_chain + c];
            bool hit = ch.is_default;
            for (int w = 0; w < PTX_MOD_WORDS && !hit; w++) hit = (mask[w] & ch.key[w]) != 0;
            if (hit) return parse_pattern(ch.pattern, mb, me, ins);
        }
        return false;
    }

    bool parse_call(Instruction& ins) {
        bool uni = eat(T_MOD_uni);
        std::vector<sv> rets;
        bool has_rets = false;
        {
            size_t save = pos;
            sv id;
            if (eat(T_LPAREN) && ident(&id)) {
                rets.push_back(id);
                for (;;) {
                    size_t s2 = pos;
                    if (!eat(T_COMMA)) break;
                    if (!ident(&id)) { pos = s2; break; }
                    rets.push_back(id);
                }
                if (eat(T_RPAREN) && eat(T_COMMA)) has_rets = true;
            }
            if (!has_rets) { pos = save; rets.clear(); }
        }
        sv name;
        if (!ident(&name)) return false;
        std::vector<int> inputs;
        {
            size_t save = pos;
            size_t nops = ins.ops.size();
            bool ok = false;
            Operand o;
            if (eat(T_COMMA) && eat(T_LPAREN) && operand(&o)) {
                ins.ops.push_back(std::move(o));
                inputs.push_back((int)ins.ops.size() - 1);
                for (;;) {
                    size_t s2 = pos;
                    if (!eat(T_COMMA)) break;
                    if (!operand(&o)) { pos = s2; break; }
                    ins.ops.push_back(std::move(o));
                    inputs.push_back((int)ins.ops.size() - 1);
                }
                if (eat(T_RPAREN)) ok = true;
            }
            if (!ok) { pos = save; ins.ops.resize(nops); inputs.clear(); }
        }
        ins.variant = I_Call;
        ins.call_uniform = uni;
        ins.call_func = name;
        auto it = fns.find(name);
        if (it == fns.end()) { push(E_UNKNOWN_FUNCTION); ins.ops.clear(); return true; }
        if (it->second.first.size() != rets.size() || it->second.second.size() != inputs.size()) {
            push(E_MALFORMED_CALL);
            ins.ops.clear();
            return true;
        }
        ins.call_ret_types = it->second.first;
        ins.call_in_types = it->second.second;
        ins.call_rets = rets;
        ins.call_inputs = inputs;
        return true;
    }

    // ---- statements, lib.rs:858-959, 1371-1431
    bool debug_directive() {
        size_t save = pos;
        uint32_t x;
        if (!(eat(T_DOT_LOC) && u32(&x) && u32(&x) && u32(&x))) { pos = save; return false; }
        size_t s2 = pos;
        sv id;
        bool ok = false;
        if (eat(T_COMMA) && ident_literal("function_name") && ident(&id)) {
            if (eat(T_COMMA)) ok = ident_literal("inlined_at") && u32(&x) && u32(&x) && u32(&x);
            else if (eat(T_PLUS)) ok = u32(&x) && eat(T_COMMA) && ident_literal("inlined_at") && u32(&x) && u32(&x) && u32(&x);
        }
        if (!ok) pos = s2;
        return true;
    }
    // take_till_end_of_statement: number of tokens to skip, or -1
    long recovery_len() const {
        int depth = 0;
        for (size_t i = pos; i < t.size(); i++) {
            uint16_t k = t[i].kind;
            if (k == T_LBRACE) depth++;
            else if (k == T_RBRACE) {
                if (depth == 0) return -1;
                depth--;
            } else if (k == T_SEMI || k == T_COLON) {
                return (i + 1 < t.size()) ? (long)(i + 1 - pos) : (long)(i - pos);
            }
        }
        return -1;
    }
    // returns false when neither the statement nor its recovery matches (the enclosing repeat stops)
    bool statement(std::vector<Statement>* out) {
        // Work budget.  A block that fails to parse is recovered from its '{' and its contents are then parsed again as
        // statements of the enclosing block (lib.rs:858-880, 921-951): damage below d levels of nesting multiplies the
        // work (and the appended errors) by 2^d, and winnow does not memoise.  Where the reference would in practice
        // not come back, parsing stops after 4 * tokens + 1024 statement attempts with the verdict ReferenceDiverges.
        if (diverged || ++attempts > 4 * (uint64_t)t.size() + 1024) { diverged = true; return false; }
        size_t save = pos;
        Statement st;
        // label
        {
            sv id;
            if (ident(&id) && eat(T_COLON)) { st.kind = 0; st.label = id; out->push_back(std::move(st)); return true; }
            pos = save;
        }
        if (debug_directive()) return true;
        pos = save;
        {
            int space = -1;
            switch (kind()) {
            case T_DOT_REG: space = StateSpace_Reg; break;
            case T_MOD_local: space = StateSpace_Local; break;
            case T_MOD_param: space = StateSpace_Param; break;
            case T_MOD_global: space = StateSpace_Global; break;
            case T_MOD_const: space = StateSpace_Const; break;
            case T_MOD_shared: space = StateSpace_Shared; break;
            default: break;
            }
            if (space >= 0) {
                pos++;
                if (multi_variable(false, space, &st.var) && eat(T_SEMI)) { st.kind = 1; out->push_back(std::move(st)); return true; }
                pos = save;
            }
        }
        {
            bool ok = true;
            if (eat(T_AT)) {
                st.pred_not = eat(T_EXCL);
                ok = ident(&st.pred);
                st.has_pred = ok;
            }
            if (!ok) { pos = save; st.has_pred = false; ok = true; }   // opt(pred_at) resets; the instruction then sees '@'
            if (parse_instruction(&st.ins) && eat(T_SEMI)) { st.kind = 2; out->push_back(std::move(st)); return true; }
            pos = save;
        }
        if (eat(T_DOT_PRAGMA) && eat(T_STRING) && eat(T_SEMI)) return true;
        pos = save;
        if (eat(T_LBRACE)) {
            Statement blk;
            blk.kind = 3;
            while (statement(&blk.block)) {}
            if (eat(T_RBRACE)) { out->push_back(std::move(blk)); return true; }
            pos = save;
        }
        long n = recovery_len();
        if (n < 0) return false;
        if (n == 0) { panicked = true; return false; }   // the reference unwraps an empty slice here
        uint32_t a = t[pos].start, b = t[pos + n - 1].end;
        pos += n;
        push(E_UNRECOGNIZED_STATEMENT, 0, a, b - a);
        return true;
    }
    bool panicked = false;
    bool diverged = false;
    uint64_t attempts = 0;

    // ---- directives, lib.rs:579-856
    static bool directive_start(uint16_t k) {
        return k == T_DOT_EXTERN || k == T_DOT_VISIBLE || k == T_MOD_weak || k == T_DOT_FUNC || k == T_DOT_ENTRY ||
               k == T_MOD_global || k == T_MOD_const || k == T_MOD_shared || k == T_DOT_FILE || k == T_DOT_SECTION;
    }
    int linking() {
        int l = 0;
        for (;;) {
            if (eat(T_DOT_EXTERN)) l |= 1;
            else if (eat(T_DOT_VISIBLE)) l |= 2;
            else if (eat(T_MOD_weak)) l |= 4;
            else break;
        }
        return l;
    }
    bool tuning(Tuning* tn) {
        size_t save = pos;
        auto tuple = [&](uint32_t* v) -> bool {
            v[0] = v[1] = v[2] = 1;
            if (!u32(&v[0])) return false;
            for (int i = 1; i < 3; i++) {
                size_t s2 = pos;
                if (!(eat(T_COMMA) && u32(&v[i]))) { pos = s2; v[i] = 1; break; }
            }
            return true;
        };
        bool ok = false;
        if (eat(T_DOT_MAXNREG)) { tn->kind = 0; ok = u32(&tn->v[0]); }
        else if (eat(T_DOT_MAXNTID)) { tn->kind = 1; ok = tuple(tn->v); }
        else if (eat(T_DOT_REQNTID)) { tn->kind = 2; ok = tuple(tn->v); }
        else if (eat(T_DOT_MINNCTAPERSM)) { tn->kind = 3; ok = u32(&tn->v[0]); }
        else if (eat(T_DOT_NORETURN)) { tn->kind = 4; ok = true; }
        if (!ok) pos = save;
        return ok;
    }
    bool function(Directive* d) {
        size_t save = pos;
        d->linking = linking();
        Function& f = d->func;
        f = Function();
        bool ok = false;
        if (eat(T_DOT_ENTRY)) {
            f.is_kernel = true;
            ok = ident(&f.name) && param_list(true, &f.inputs);
        } else if (eat(T_DOT_FUNC)) {
            if (!param_list(false, &f.rets)) f.rets.clear();
            ok = ident(&f.name) && param_list(false, &f.inputs);
        }
        if (!ok) { pos = save; return false; }
        Tuning tn;
        while (tuning(&tn)) f.tuning.push_back(tn);
        if (eat(T_LBRACE)) {
            f.has_body = true;
            while (statement(&f.body)) {}
            if (!eat(T_RBRACE)) { pos = save; return false; }
        } else if (!eat(T_SEMI)) {
            pos = save;
            return false;
        }
        std::vector<TypeSpace> r, in;
        for (auto& v : f.rets) r.push_back({v.info.type, v.info.space});
        for (auto& v : f.inputs) in.push_back({v.info.type, v.info.space});
        fns[f.name] = {std::move(r), std::move(in)};
        d->is_method = true;
        return true;
    }
    bool file_directive() {
        size_t save = pos;
        uint32_t x;
        if (!(eat(T_DOT_FILE) && u32(&x) && eat(T_STRING))) { pos = save; return false; }
        size_t s2 = pos;
        if (!(eat(T_COMMA) && u32(&x) && eat(T_COMMA) && u32(&x))) pos = s2;
        return true;
    }
    bool section_label() {
        sv id;
        return ident(&id) || dot_ident(&id);
    }
    bool section_directive() {
        size_t save = pos;
        sv name;
        if (!(eat(T_DOT_SECTION) && dot_ident(&name) && eat(T_LBRACE))) { pos = save; return false; }
        for (;;) {
            size_t s2 = pos;
            uint32_t x;
            if (section_label() && eat(T_COLON)) continue;
            pos = s2;
            if ((eat(T_MOD_b32) || eat(T_MOD_b64)) && section_label()) {
                size_t s3 = pos;
                if (!(eat(T_OP_ADD) && u32(&x))) pos = s3;
                continue;
            }
            pos = s2;
            if ((eat(T_MOD_b8) || eat(T_MOD_b16) || eat(T_MOD_b32) || eat(T_MOD_b64)) && u32(&x)) {
                for (;;) {
                    size_t s3 = pos;
                    if (!(eat(T_COMMA) && u32(&x))) { pos = s3; break; }
                }
                continue;
            }
            pos = s2;
            break;
        }
        if (!eat(T_RBRACE)) { pos = save; return false; }
        return true;
    }
    bool module_variable(Directive* d) {
        size_t save = pos;
        d->linking = linking();
        int space = -1;
        if (eat(T_MOD_global)) space = StateSpace_Global;
        else if (eat(T_MOD_const)) space = StateSpace_Const;
        else if (eat(T_MOD_shared)) space = StateSpace_Shared;
        MultiVar mv;
        if (space < 0 || !multi_variable((d->linking & 1) != 0, space, &mv) || mv.parameterized || mv.names.size() != 1 ||
            !eat(T_SEMI)) {
            pos = save;
            return false;
        }
        d->is_method = false;
        d->var.info = std::move(mv.info);
        d->var.name = mv.names[0];
        return true;
    }
    // 0 = stop (no directive, no recovery), 1 = directive kept, 2 = parsed but produces nothing, 3 = invalid
    int directive(Directive* d) {
        size_t nerr = errors.size();
        size_t save = pos;
        int r = 0;
        if (function(d)) r = 1;
        else if (pos = save, file_directive()) r = 2;
        else if (pos = save, section_directive()) r = 2;
        else if (pos = save, module_variable(d)) r = 1;
        else {
            pos = save;
            if (eof()) return 0;
            size_t i = pos + 1;
            while (i < t.size() && !directive_start(t[i].kind)) i++;
            if (i == pos + 1) return 0;   // take_till(1..) needs at least one token
            uint32_t a = t[pos].start, b = t[i - 1].end;
            pos = i;
            push(E_UNRECOGNIZED_DIRECTIVE, 0, a, b - a);
            r = 3;
        }
        if (errors.size() != nerr) return 3;
        return r;
    }
    bool module(Module* m) {
        Imm v;
        if (!(eat(T_DOT_VERSION) && f64_tok(&v))) return false;
        double ver;
        memcpy(&ver, &v.bits, 8);
        auto sat_u8 = [](double x) -> uint8_t { return !(x > 0) ? 0 : x >= 255 ? 255 : (uint8_t)x; };
        m->major = sat_u8(std::floor(ver));
        m->minor = sat_u8(std::round((ver - std::floor(ver)) * 10.0));
        if (!eat(T_DOT_TARGET)) return false;
        sv tgt;
        if (!ident(&tgt)) return false;
        {
            // shader_model: "sm_" dec_uint [a-z]? eof   (lib.rs:561-570)
            if (tgt.size() < 4 || tgt.substr(0, 3) != "sm_") return false;
            size_t i = 3;
            uint64_t n = 0;
            if (!is_digit(tgt[i])) return false;
            while (i < tgt.size() && is_digit(tgt[i])) {
                n = n * 10 + (tgt[i] - '0');
                if (n > UINT32_MAX) return false;
                i++;
            }
            if (i < tgt.size() && tgt[i] >= 'a' && tgt[i] <= 'z') i++;
            if (i != tgt.size()) return false;
            m->sm = (uint32_t)n;
        }
        {
            size_t s2 = pos;
            if (!(eat(T_COMMA) && ident_literal("debug"))) pos = s2;
        }
        m->address_size = 32;
        {
            size_t s2 = pos;
            bool ok = false;
            if (eat(T_DOT_ADDRESS_SIZE)) {
                size_t s3 = pos;
                uint32_t x;
                if (u8(&x) && x == 64) { m->address_size = 64; ok = true; }
                else {
                    pos = s3;
                    if (u8(&x) && x == 32) { m->address_size = 32; ok = true; }
                }
            }
            if (!ok) pos = s2;
        }
        for (;;) {
            Directive d;
            int r = directive(&d);
            if (r == 0 || diverged) break;
            if (r == 1) m->directives.push_back(std::move(d));
            else if (r == 3) m->invalid++;
        }
        return eof();
    }
};

// =============================================================================================== canonical dump
struct Out {
    std::string s;
    // hash-only mode: the text is folded into a 64-bit FNV-1a hash as it grows and is not kept (a module with millions of
    // initialisers dumps to gigabytes)
    bool hashing = false;
    uint64_t h = 1469598103934665603ull;
    void fold() {
        for (unsigned char c : s) h = (h ^ c) * 1099511628211ull;
        s.clear();
    }
    void tick() { if (hashing && s.size() > (1u << 16)) fold(); }
    void put(sv x) { s.append(x); tick(); }
    void putf(const char* fmt, ...) __attribute__((format(printf, 2, 3))) {
        char buf[128];
        va_list ap;
        va_start(ap, fmt);
        int n = vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        s.append(buf, n);
    }
    void str(sv x) {
        s.push_back('"');
        for (unsigned char c : x) {
            if (c == '"') s += "\\\"";
            else if (c == '\\') s += "\\\\";
            else if (c == '\n') s += "\\n";
            else if (c == '\r') s += "\\r";
            else if (c == '\t') s += "\\t";
            else if (c < 0x20 || c == 0x7f) putf("\\u{%x}", c);
            else s.push_back((char)c);
        }
        s.push_back('"');
    }
    void indent(int d) { s.append((size_t)d * 2, ' '); }
};

void dump_imm(Out& o, const Imm& i) {
    switch (i.kind) {
    case 0: o.putf("U64(%llu)", (unsigned long long)i.bits); break;
    case 1: o.putf("S64(%lld)", (long long)i.bits); break;
    case 2: o.putf("F32(bits=0x%08X)", (unsigned)i.bits); break;
    default: o.putf("F64(bits=0x%016llX)", (unsigned long long)i.bits); break;
    }
}
void dump_roi(Out& o, const RegOrImm& r) {
    if (r.is_reg) { o.put("Reg("); o.str(r.reg); o.put(")"); }
    else { o.put("Imm("); dump_imm(o, r.imm); o.put(")"); }
}
void dump_operand(Out& o, const Operand& p) {
    switch (p.kind) {
    case 0: o.put("Reg("); o.str(p.name); o.put(")"); break;
    case 1: o.put("RegOffset("); o.str(p.name); o.putf(", %d)", p.offset); break;
    case 2: o.put("Imm("); dump_imm(o, p.imm); o.put(")"); break;
    case 3: o.put("VecMember("); o.str(p.name); o.putf(", %u)", p.index); break;
    default:
        o.put("VecPack([");
        for (size_t i = 0; i < p.pack.size(); i++) {
            if (i) o.put(", ");
            dump_roi(o, p.pack[i]);
        }
        o.put("])");
        break;
    }
}
void dump_type(Out& o, const Type& ty) {
    switch (ty.kind) {
    case 0: o.putf("Scalar(%s)", ScalarType_names[ty.scalar]); break;
    case 1: o.putf("Vector(%d, %s)", ty.vec, ScalarType_names[ty.scalar]); break;
    case 2:
        if (ty.vec) o.putf("Array(Some(%d), %s, [", ty.vec, ScalarType_names[ty.scalar]);
        else o.putf("Array(None, %s, [", ScalarType_names[ty.scalar]);
        for (size_t i = 0; i < ty.dims.size(); i++) o.putf(i ? ", %u" : "%u", ty.dims[i]);
        o.put("])");
        break;
    default: o.put("Texref"); break;
    }
}
void dump_info(Out& o, const VarInfo& v) {
    if (v.has_align) o.putf("VariableInfo { align: Some(%u), v_type: ", v.align);
    else o.put("VariableInfo { align: None, v_type: ");
    dump_type(o, v.type);
    o.putf(", state_space: %s, array_init: [", StateSpace_names[v.space]);
    for (size_t i = 0; i < v.init.size(); i++) {
        if (i) o.put(", ");
        dump_roi(o, v.init[i]);
    }
    o.put("] }");
}
void dump_variable(Out& o, const Variable& v) {
    o.put("Variable { info: ");
    dump_info(o, v.info);
    o.put(", name: ");
    o.str(v.name);
    o.put(" }");
}

// schema-driven dump of an instruction's data words
void dump_schema(Out& o, int type, const uint32_t*& w) {
    const PtxType& ty = ptx_types[type];
    switch (ty.kind) {
    case 0:
        switch (ty.a) {
        case 0: o.put(*w++ ? "true" : "false"); break;
        case 3: { uint64_t v = w[0] | ((uint64_t)w[1] << 32); w += 2; o.putf("%llu", (unsigned long long)v); break; }
        case 4: o.putf("bits=0x%08X", *w++); break;
        default: o.putf("%u", *w++); break;
        }
        break;
    case 1: o.put(ptx_enum_names[type][*w++]); break;
    case 2:
        o.put(ty.name);
        if (ty.b) {
            o.put(" { ");
            for (int i = 0; i < ty.b; i++) {
                if (i) o.put(", ");
                o.put(ptx_fields[ty.a + i].name);
                o.put(": ");
                dump_schema(o, ptx_fields[ty.a + i].type, w);
            }
            o.put(" }");
        }
        break;
    case 3: {
        const PtxVariant& v = ptx_variants[ty.a + *w++];
        o.put(v.name);
        if (v.n_fields) {
            o.put(v.named ? " { " : "(");
            for (int i = 0; i < v.n_fields; i++) {
                if (i) o.put(", ");
                if (v.named) { o.put(ptx_fields[v.first_field + i].name); o.put(": "); }
                dump_schema(o, ptx_fields[v.first_field + i].type, w);
            }
            o.put(v.named ? " }" : ")");
        }
        break;
    }
    default:
        if (*w++) { o.put("Some("); dump_schema(o, ty.a, w); o.put(")"); }
        else o.put("None");
        break;
    }
}

bool g_schema_ok = true;

void dump_instruction(Out& o, const Instruction& ins) {
    const PtxInstr& in = ptx_instrs[ins.variant];
    o.put(in.name);
    if (ins.variant == I_Bra) {
        o.put(" { arguments: BraArgs { src: ");
        o.str(ins.bra_target);
        o.put(" } }");
        return;
    }
    if (ins.variant == I_Call) {
        o.putf(" { data: CallDetails { uniform: %s, return_arguments: [", ins.call_uniform ? "true" : "false");
        for (size_t i = 0; i < ins.call_ret_types.size(); i++) {
            o.put(i ? ", (" : "(");
            dump_type(o, ins.call_ret_types[i].type);
            o.putf(", %s)", StateSpace_names[ins.call_ret_types[i].space]);
        }
        o.put("], input_arguments: [");
        for (size_t i = 0; i < ins.call_in_types.size(); i++) {
            o.put(i ? ", (" : "(");
            dump_type(o, ins.call_in_types[i].type);
            o.putf(", %s)", StateSpace_names[ins.call_in_types[i].space]);
        }
        o.put("] }, arguments: CallArgs { return_arguments: [");
        for (size_t i = 0; i < ins.call_rets.size(); i++) {
            if (i) o.put(", ");
            o.str(ins.call_rets[i]);
        }
        o.put("], func: ");
        o.str(ins.call_func);
        o.put(", input_arguments: [");
        for (size_t i = 0; i < ins.call_inputs.size(); i++) {
            if (i) o.put(", ");
            dump_operand(o, ins.ops[ins.call_inputs[i]]);
        }
        o.put("], is_external: false } }");
        return;
    }
    if (in.data_type < 0 && in.n_args == 0) return;
    o.put(" { ");
    if (in.data_type >= 0) {
        o.put("data: ");
        const uint32_t* w = ins.data.data();
        if (ptx_types[in.data_type].kind == 2 && ptx_types[in.data_type].b == 0) o.put("()");
        else dump_schema(o, in.data_type, w);
        if (w != ins.data.data() + ins.data.size()) g_schema_ok = false;
        if (in.n_args) o.put(", ");
    }
    if (in.n_args) {
        o.putf("arguments: %sArgs { ", in.name);
        if ((int)ins.args.size() != in.n_args) g_schema_ok = false;
        for (int i = 0; i < in.n_args && i < (int)ins.args.size(); i++) {
            if (i) o.put(", ");
            const PtxArg& a = ptx_args[in.first_arg + i];
            o.put(a.name);
            o.put(": ");
            int ref = ins.args[i];
            if (a.optional) {
                if (ref < 0) o.put("None");
                else { o.put("Some("); dump_operand(o, ins.ops[ref]); o.put(")"); }
            } else if (ref < 0) {
                g_schema_ok = false;
                o.put("<missing>");
            } else {
                dump_operand(o, ins.ops[ref]);
            }
        }
        o.put(" }");
    }
    o.put(" }");
}

void dump_statements(Out& o, const std::vector<Statement>& v, int depth) {
    for (const Statement& st : v) {
        o.indent(depth);
        switch (st.kind) {
        case 0: o.put("Label("); o.str(st.label); o.put(")\n"); break;
        case 1:
            if (st.var.parameterized) {
                o.put("Variable(Parameterized { info: ");
                dump_info(o, st.var.info);
                o.put(", name: ");
                o.str(st.var.names[0]);
                o.putf(", count: %u })\n", st.var.count);
            } else {
                o.put("Variable(Names { info: ");
                dump_info(o, st.var.info);
                o.put(", names: [");
                for (size_t i = 0; i < st.var.names.size(); i++) {
                    if (i) o.put(", ");
                    o.str(st.var.names[i]);
                }
                o.put("] })\n");
            }
            break;
        case 2:
            o.put("Instruction(");
            if (st.has_pred) { o.putf("Some(PredAt { not: %s, label: ", st.pred_not ? "true" : "false"); o.str(st.pred); o.put(" }), "); }
            else o.put("None, ");
            dump_instruction(o, st.ins);
            o.put(")\n");
            break;
        default:
            o.put("Block([\n");
            dump_statements(o, st.block, depth + 1);
            o.indent(depth);
            o.put("])\n");
            break;
        }
    }
}

void dump_module(Out& o, const Module& m) {
    o.putf("Module { ptx_version: (%u, %u), sm_version: %u, address_size: %u, invalid_directives: %llu, directives: %zu }\n",
           m.major, m.minor, m.sm, m.address_size, (unsigned long long)m.invalid, m.directives.size());
    for (const Directive& d : m.directives) {
        if (!d.is_method) {
            o.putf("Variable(LinkingDirective(%d), ", d.linking);
            dump_variable(o, d.var);
            o.put(")\n");
            continue;
        }
        const Function& f = d.func;
        o.putf("Method(LinkingDirective(%d), Function { func_directive: MethodDeclaration { return_arguments: [", d.linking);
        for (size_t i = 0; i < f.rets.size(); i++) {
            if (i) o.put(", ");
            dump_variable(o, f.rets[i]);
        }
        o.put(f.is_kernel ? "], name: Kernel(" : "], name: Func(");
        o.str(f.name);
        o.put("), input_arguments: [");
        for (size_t i = 0; i < f.inputs.size(); i++) {
            if (i) o.put(", ");
            dump_variable(o, f.inputs[i]);
        }
        o.put("], shared_mem: None }, tuning: [");
        for (size_t i = 0; i < f.tuning.size(); i++) {
            if (i) o.put(", ");
            const Tuning& tn = f.tuning[i];
            switch (tn.kind) {
            case 0: o.putf("MaxNReg(%u)", tn.v[0]); break;
            case 1: o.putf("MaxNtid(%u, %u, %u)", tn.v[0], tn.v[1], tn.v[2]); break;
            case 2: o.putf("ReqNtid(%u, %u, %u)", tn.v[0], tn.v[1], tn.v[2]); break;
            case 3: o.putf("MinNCtaPerSm(%u)", tn.v[0]); break;
            default: o.put("NoReturn"); break;
            }
        }
        if (!f.has_body) {
            o.put("], body: None })\n");
            continue;
        }
        o.put("], body: Some([\n");
        dump_statements(o, f.body, 1);
        o.put("]) })\n");
    }
}

const char* const kErrNames[] = {"ParseInt", "ParseFloat", "Lexer", "Parser", "Todo", "SyntaxError", "NonF32Ftz",
                                 "Unsupported32Bit", "WrongType", "UnknownFunction", "MalformedCall", "WrongArrayType",
                                 "WrongVectorElement", "MultiArrayVariable", "ZeroDimensionArray", "ArrayInitalizer",
                                 "NonExternPointer", "UnrecognizedStatement", "UnrecognizedDirective", "UnsupportedSreg"};
const char* const kIntErr[] = {"Empty", "InvalidDigit", "PosOverflow", "NegOverflow"};

void dump_errors(Out& o, const std::vector<Error>& errs, const char* text) {
    o.putf("errors: %zu\n", errs.size());
    for (const Error& e : errs) {
        o.put(kErrNames[e.kind]);
        switch (e.kind) {
        case E_PARSE_INT: o.putf("(%s)", kIntErr[e.sub]); break;
        case E_LEXER: o.putf("(start=%u)", e.a); break;
        case E_PARSER: o.put("(ContextError)"); break;
        case E_TODO: o.put("("); o.str(ptx_todo_msgs[e.sub]); o.put(")"); break;
        case E_SYNTAX:
            switch (e.sub) {
            case SYN_LD_NC_BOTH:
                o.putf("(\"cannot have both %s and %s in <text>\")", RawLdCacheOperator_text[e.a], EvictionPriority_text[e.b]);
                break;
            case SYN_CP_SIZE: o.put("(\"invalid cp.async cp-size "); o.put(sv(text + e.a, e.b)); o.put(" in <text>\")"); break;
            case SYN_CVT_MISSING_RND: o.put("(\"missing rounding mode for cvt\")"); break;
            case SYN_CVT_RND_ON_EXTEND: o.put("(\"should not have rounding mode when dst is larger than src in cvt\")"); break;
            default: o.put("(\"unexpected pairing of dst and src types in cvt\")"); break;
            }
            break;
        case E_UNRECOGNIZED_STATEMENT:
        case E_UNRECOGNIZED_DIRECTIVE:
        case E_UNSUPPORTED_SREG: o.put("("); o.str(sv(text + e.a, e.b)); o.put(")"); break;
        default: break;
        }
        o.put("\n");
    }
}

enum { MODE_CHECKED = 0, MODE_UNCHECKED = 1, MODE_ERRORS_ONLY = 2 };

// lib.rs:392-501.  The dump has a fixed layout: mode line, status line, the module (when one is returned), the errors.
// With `hash_out` the dump is not kept: its FNV-1a hash is returned there and the string comes back empty.
std::string run(const char* text, size_t n, int mode, int* status, uint64_t* hash_out = nullptr) {
    LexResult lx = lex(text, n);
    std::vector<Error> errors;
    for (const Tok& e : lx.errors) errors.push_back({E_LEXER, 0, e.start, e.end - e.start});
    Out o;
    o.hashing = hash_out != nullptr;
    Module m;
    bool have_module = false;
    const char* verdict;
    bool panicked = false;
    if (!lx.errors.empty() && mode != MODE_ERRORS_ONLY) {
        verdict = mode == MODE_CHECKED ? "Err" : "Empty";
    } else {
        Parser p(text, n, lx.toks, errors);
        bool ok = p.module(&m);
        panicked = p.panicked;
        if (p.diverged) {
            o.putf("mode: %s\nstatus: ReferenceDiverges\nerrors: 0\n", mode == MODE_CHECKED ? "checked" : mode == MODE_UNCHECKED ? "unchecked" : "errors");
            *status = 1;
            if (hash_out) { o.fold(); *hash_out = o.h; }
            return std::move(o.s);
        }
        if (!ok) errors.push_back({E_PARSER, 0, 0, 0});
        if (mode == MODE_CHECKED) {
            have_module = ok && errors.empty() && m.invalid == 0;
            verdict = have_module ? "Ok" : "Err";
        } else if (mode == MODE_UNCHECKED) {
            have_module = ok;
            verdict = ok ? "Module" : "Empty";
        } else {
            verdict = "Errors";
        }
    }
    if (panicked) verdict = "ReferencePanics";
    o.putf("mode: %s\nstatus: %s\n", mode == MODE_CHECKED ? "checked" : mode == MODE_UNCHECKED ? "unchecked" : "errors", verdict);
    if (have_module) dump_module(o, m);
    else if (mode == MODE_UNCHECKED)
        o.put("Module { ptx_version: (1, 0), sm_version: 0, address_size: 64, invalid_directives: 18446744073709551615, directives: 0 }\n");
    dump_errors(o, errors, text);
    *status = have_module ? 0 : 1;
    if (hash_out) { o.fold(); *hash_out = o.h; }
    return std::move(o.s);
}

}   // namespace

// =============================================================================================== C entry points (tests, CPU baseline)
extern "C" {

// Parse one module and return the canonical dump (malloc'ed, NUL-terminated; free with oracle_free).
char* oracle_parse(const char* text, uint64_t len, int mode, uint64_t* out_len, int* status) {
    int st = 0;
    std::string s = run(text, len, mode, &st);
    char* r = (char*)malloc(s.size() + 1);
    memcpy(r, s.data(), s.size() + 1);
    if (out_len) *out_len = s.size();
    if (status) *status = st;
    return r;
}

// 64-bit FNV-1a of the canonical dump (parity checks over many large modules: the dump itself stays on this side).
uint64_t oracle_dump_hash(const char* text, uint64_t len, int mode, int* status) {
    int st = 0;
    uint64_t h = 0;
    run(text, len, mode, &st, &h);
    if (status) *status = st;
    return h;
}

// Parse without producing the dump (the timed CPU baseline).  Returns 0 when parse_module_checked would be Ok.
int oracle_parse_only(const char* text, uint64_t len, uint64_t* n_tokens, uint64_t* n_errors) {
    LexResult lx = lex(text, len);
    std::vector<Error> errors;
    if (n_tokens) *n_tokens = lx.toks.size();
    if (!lx.errors.empty()) {
        if (n_errors) *n_errors = lx.errors.size();
        return 1;
    }
    Parser p(text, len, lx.toks, errors);
    Module m;
    bool ok = p.module(&m);
    if (n_errors) *n_errors = errors.size();
    return (ok && errors.empty() && m.invalid == 0) ? 0 : 1;
}

// Token list: triples (kind, start, length) as uint32, then error spans (start, length).
uint32_t* oracle_lex(const char* text, uint64_t len, uint64_t* n_tokens, uint64_t* n_errors) {
    LexResult lx = lex(text, len);
    uint32_t* r = (uint32_t*)malloc((lx.toks.size() * 3 + lx.errors.size() * 2 + 1) * 4);
    size_t k = 0;
    for (const Tok& t : lx.toks) { r[k++] = t.kind; r[k++] = t.start; r[k++] = t.end - t.start; }
    for (const Tok& t : lx.errors) { r[k++] = t.start; r[k++] = t.end - t.start; }
    *n_tokens = lx.toks.size();
    *n_errors = lx.errors.size();
    return r;
}

int oracle_schema_ok() { return g_schema_ok ? 1 : 0; }
// Coverage of the instruction patterns by everything parsed since the last reset: out[i] = 1 if pattern i matched.
int oracle_pattern_count() { return PTX_N_PATTERNS; }
const char* oracle_pattern_head(int i) { return i >= 0 && i < PTX_N_PATTERNS ? ptx_pattern_heads[i] : ""; }
void oracle_pattern_hits(unsigned char* out, int reset) {
    for (int i = 0; i < PTX_N_PATTERNS; i++) {
        if (out) out[i] = g_pattern_hits[i];
        if (reset) g_pattern_hits[i] = 0;
    }
}
const char* oracle_token_text(int kind) { return kind >= 0 && kind < T_COUNT ? ptx_tok_text[kind] : ""; }
int oracle_token_count() { return T_COUNT; }
void oracle_free(void* p) { free(p); }
}
