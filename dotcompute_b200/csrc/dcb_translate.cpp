// dcb_translate.cpp — see dcb_translate.h.
#include "dcb_translate.h"

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>

namespace dcbt {

// Operator and status codes shared with dcb200.h (kept numeric here so this file has no CUDA dependency).
enum { OP_SELECT = 1, OP_WHERE = 2, OP_ZIP = 3, OP_TOARRAY = 16, OP_SUM = 17, OP_MIN = 18, OP_MAX = 19, OP_AVERAGE = 20, OP_COUNT = 21,
       OP_FIRST_INDEX = 22, OP_LAST_INDEX = 23 };
enum { ST_INVALID_ARGUMENT = 301, ST_NOT_SUPPORTED = 302 };
enum { RED_SUM = 1, RED_MIN = 2, RED_MAX = 4, RED_COUNT = 8, RED_FIRST = 16, RED_LAST = 32 };

static const char* kCuda[] = {"void", "signed char", "unsigned char", "short", "unsigned short", "int", "unsigned int",
                              "long long", "unsigned long long", "float", "double", "bool"};
static const char* kCs[] = {"void", "sbyte", "byte", "short", "ushort", "int", "uint", "long", "ulong", "float", "double", "bool"};
static const int kSize[] = {0, 1, 1, 2, 2, 4, 4, 8, 8, 4, 8, 1};

const char* cuda_name(int t) { return (t >= 0 && t <= T_BOOL) ? kCuda[t] : "void"; }
const char* csharp_name(int t) { return (t >= 0 && t <= T_BOOL) ? kCs[t] : "void"; }
int type_size(int t) { return (t >= 0 && t <= T_BOOL) ? kSize[t] : 0; }
bool is_numeric(int t) { return t >= T_I8 && t <= T_F64; }
static bool is_integral(int t) { return t >= T_I8 && t <= T_U64; }
static bool is_signed_int(int t) { return t == T_I8 || t == T_I16 || t == T_I32 || t == T_I64; }
static bool is_float(int t) { return t == T_F32 || t == T_F64; }
static int unsigned_of(int t) { return t == T_I32 ? T_U32 : t == T_I64 ? T_U64 : t; }

unsigned long long fnv1a(const std::string& s) {
    unsigned long long h = 1469598103934665603ull;
    for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
    return h;
}

// ---------------------------------------------------------------------------------------------- tokens
struct Tok {
    enum Kind { END, NUM, IDENT, PUNCT } kind = END;
    std::string text;
};

static bool lex(const std::string& s, std::vector<Tok>* out, std::string* err) {
    size_t i = 0, n = s.size();
    while (i < n) {
        char c = s[i];
        if (isspace((unsigned char)c)) { ++i; continue; }
        Tok t;
        if (isdigit((unsigned char)c) || (c == '.' && i + 1 < n && isdigit((unsigned char)s[i + 1]))) {
            size_t j = i;
            bool hex = (c == '0' && j + 1 < n && (s[j + 1] == 'x' || s[j + 1] == 'X'));
            bool bin = (c == '0' && j + 1 < n && (s[j + 1] == 'b' || s[j + 1] == 'B'));
            if (hex || bin) {
                j += 2;
                while (j < n && (isxdigit((unsigned char)s[j]) || s[j] == '_')) ++j;
            } else {
                while (j < n && (isdigit((unsigned char)s[j]) || s[j] == '_')) ++j;
                if (j < n && s[j] == '.' && j + 1 < n && isdigit((unsigned char)s[j + 1])) {
                    ++j;
                    while (j < n && (isdigit((unsigned char)s[j]) || s[j] == '_')) ++j;
                }
                if (j < n && (s[j] == 'e' || s[j] == 'E')) {
                    size_t k = j + 1;
                    if (k < n && (s[k] == '+' || s[k] == '-')) ++k;
                    if (k < n && isdigit((unsigned char)s[k])) {
                        j = k;
                        while (j < n && isdigit((unsigned char)s[j])) ++j;
                    }
                }
            }
            while (j < n && isalpha((unsigned char)s[j])) ++j;   // suffix
            t.kind = Tok::NUM; t.text = s.substr(i, j - i); i = j;
        } else if (isalpha((unsigned char)c) || c == '_' || c == '@') {
            size_t j = i + 1;
            while (j < n && (isalnum((unsigned char)s[j]) || s[j] == '_')) ++j;
            t.kind = Tok::IDENT; t.text = s.substr(i, j - i); i = j;
        } else {
            static const char* three[] = {">>>", "<<=", ">>=", nullptr};
            static const char* two[] = {"=>", "==", "!=", "<=", ">=", "&&", "||", "<<", ">>", "+=", "-=", "*=", "/=", "%=", "&=", "|=", "^=", "++", "--", nullptr};
            t.kind = Tok::PUNCT;
            bool done = false;
            if (s.compare(i, 4, ">>>=") == 0) { t.text = ">>>="; i += 4; done = true; }
            for (int k = 0; three[k] && !done; ++k)
                if (s.compare(i, 3, three[k]) == 0) { t.text = three[k]; i += 3; done = true; }
            for (int k = 0; two[k] && !done; ++k)
                if (s.compare(i, 2, two[k]) == 0) { t.text = two[k]; i += 2; done = true; }
            if (!done) {
                if (strchr("+-*/%&|^~!<>?:(),.;{}[]=", c) == nullptr) { *err = std::string("unexpected character '") + c + "'"; return false; }
                t.text = std::string(1, c); ++i;
            }
        }
        out->push_back(t);
    }
    out->push_back(Tok());
    return true;
}

// ---------------------------------------------------------------------------------------------- typed nodes
struct Node {
    std::string code;
    int type = T_NONE;
    bool const_int = false;       // an int-typed constant expression (C# lets it narrow implicitly when it fits)
    long long cval = 0;
    bool is_buffer = false;       // a Span<T> / T[] kernel parameter: `type` is its element type, only a[i] and a.Length are allowed
    bool is_lvalue = false;       // may stand on the left of an assignment
};

static std::string conv(const Node& n, int to) {
    if (n.type == to) return n.code;
    return std::string("((") + cuda_name(to) + ")(" + n.code + "))";
}

// C# implicit numeric conversions (from -> to).
static bool implicit_ok(int from, int to) {
    if (from == to) return true;
    switch (from) {
        case T_I8: return to == T_I16 || to == T_I32 || to == T_I64 || to == T_F32 || to == T_F64;
        case T_U8: return to == T_I16 || to == T_U16 || to == T_I32 || to == T_U32 || to == T_I64 || to == T_U64 || to == T_F32 || to == T_F64;
        case T_I16: return to == T_I32 || to == T_I64 || to == T_F32 || to == T_F64;
        case T_U16: return to == T_I32 || to == T_U32 || to == T_I64 || to == T_U64 || to == T_F32 || to == T_F64;
        case T_I32: return to == T_I64 || to == T_F32 || to == T_F64;
        case T_U32: return to == T_I64 || to == T_U64 || to == T_F32 || to == T_F64;
        case T_I64: case T_U64: return to == T_F32 || to == T_F64;
        case T_F32: return to == T_F64;
        default: return false;
    }
}

static bool const_fits(long long v, int t) {
    switch (t) {
        case T_I8: return v >= -128 && v <= 127;
        case T_U8: return v >= 0 && v <= 255;
        case T_I16: return v >= -32768 && v <= 32767;
        case T_U16: return v >= 0 && v <= 65535;
        case T_U32: return v >= 0 && v <= 4294967295LL;
        case T_U64: return v >= 0;
        default: return false;
    }
}

// Binary numeric promotion (ECMA-334 12.4.7.3). Returns T_NONE when C# would reject the pair.
static int promote_binary(const Node& a, const Node& b) {
    int x = a.type, y = b.type;
    if (!is_numeric(x) || !is_numeric(y)) return T_NONE;
    if (x == T_F64 || y == T_F64) return T_F64;
    if (x == T_F32 || y == T_F32) return T_F32;
    if (x == T_U64 || y == T_U64) {
        int o = (x == T_U64) ? y : x;
        const Node& on = (x == T_U64) ? b : a;
        if (is_signed_int(o) && !(on.const_int && on.cval >= 0)) return T_NONE;
        return T_U64;
    }
    if (x == T_I64 || y == T_I64) return T_I64;
    if (x == T_U32 || y == T_U32) {
        int o = (x == T_U32) ? y : x;
        const Node& on = (x == T_U32) ? b : a;
        if (is_signed_int(o)) return (on.const_int && on.cval >= 0) ? T_U32 : T_I64;
        return T_U32;
    }
    return T_I32;
}
static int promote_unary(int t) { return (t == T_I8 || t == T_U8 || t == T_I16 || t == T_U16) ? T_I32 : t; }

// Best common type of two operands of ?: / Math.Min / Math.Max / Math.Clamp.
static int common_type(const Node& a, const Node& b) {
    if (a.type == b.type) return a.type;
    if (a.const_int && const_fits(a.cval, b.type)) return b.type;
    if (b.const_int && const_fits(b.cval, a.type)) return a.type;
    if (implicit_ok(a.type, b.type)) return b.type;
    if (implicit_ok(b.type, a.type)) return a.type;
    return T_NONE;
}

static std::string fmt_f32(float v) {
    char buf[64];
    if (std::isnan(v)) return "__int_as_float(0x7fc00000)";
    if (std::isinf(v)) return v > 0 ? "__int_as_float(0x7f800000)" : "__int_as_float(0xff800000)";
    snprintf(buf, sizeof buf, "%.9g", (double)v);
    std::string s = buf;
    if (s.find_first_of(".en") == std::string::npos) s += ".0";
    return s + "f";
}
static std::string fmt_f64(double v) {
    char buf[64];
    if (std::isnan(v)) return "__longlong_as_double(0x7ff8000000000000LL)";
    if (std::isinf(v)) return v > 0 ? "__longlong_as_double(0x7ff0000000000000LL)" : "__longlong_as_double(0xfff0000000000000LL)";
    snprintf(buf, sizeof buf, "%.17g", v);
    std::string s = buf;
    if (s.find_first_of(".en") == std::string::npos) s += ".0";
    return s;
}

// ---------------------------------------------------------------------------------------------- parser
class Parser {
  public:
    Parser(const std::vector<Tok>& toks, const std::map<std::string, Node>& params) : t_(toks), params_(params) {}
    bool parse(Node* out, std::string* err) {
        bool ok = ternary(out) && expect_end();
        if (!ok) *err = err_.empty() ? "syntax error" : err_;
        return ok;
    }
    // Parse one expression starting at pos_ and stop behind it (statement parsers look at the delimiter themselves).
    bool parse_expr(Node* out, std::string* err) {
        bool ok = ternary(out);
        if (!ok) *err = err_.empty() ? "syntax error" : err_;
        return ok;
    }
    bool binop(const std::string& op, const Node& a, const Node& b, Node* r, std::string* err) {
        bool ok = apply_binary(op, a, b, r);
        if (!ok) *err = err_.empty() ? "bad operands" : err_;
        return ok;
    }
    size_t pos_ = 0;
    bool kernel_mode = false;        // accept KernelContext.* and buffer.Length
    bool thread_id_is_global = false; // ThreadId.X means the global index (body never names BlockId / BlockDim / GridDim)
    bool used_length = false;
    int max_dim = 1;

  private:
    const std::vector<Tok>& t_;
    const std::map<std::string, Node>& params_;
    std::string err_;

    const Tok& peek(size_t k = 0) const { return t_[std::min(pos_ + k, t_.size() - 1)]; }
    bool is_punct(const char* p, size_t k = 0) const { return peek(k).kind == Tok::PUNCT && peek(k).text == p; }
    bool accept(const char* p) { if (is_punct(p)) { ++pos_; return true; } return false; }
    bool fail(const std::string& m) { if (err_.empty()) err_ = m; return false; }
    bool expect(const char* p) { return accept(p) ? true : fail(std::string("expected '") + p + "' near '" + peek().text + "'"); }
    bool expect_end() { return peek().kind == Tok::END ? true : fail("unexpected '" + peek().text + "'"); }

    static int type_keyword(const std::string& s) {
        static const std::map<std::string, int> m = {
            {"sbyte", T_I8}, {"byte", T_U8}, {"short", T_I16}, {"ushort", T_U16}, {"int", T_I32}, {"uint", T_U32},
            {"long", T_I64}, {"ulong", T_U64}, {"float", T_F32}, {"double", T_F64}, {"bool", T_BOOL},
            {"SByte", T_I8}, {"Byte", T_U8}, {"Int16", T_I16}, {"UInt16", T_U16}, {"Int32", T_I32}, {"UInt32", T_U32},
            {"Int64", T_I64}, {"UInt64", T_U64}, {"Single", T_F32}, {"Double", T_F64}, {"Boolean", T_BOOL}};
        auto it = m.find(s);
        return it == m.end() ? T_NONE : it->second;
    }

    bool ternary(Node* out) {
        Node c;
        if (!binary(0, &c)) return false;
        if (!accept("?")) { *out = c; return true; }
        if (c.type != T_BOOL) return fail("condition of ?: must be bool");
        Node a, b;
        if (!ternary(&a) || !expect(":") || !ternary(&b)) return false;
        int t = common_type(a, b);
        if (t == T_NONE) return fail(std::string("no common type for ?: between ") + csharp_name(a.type) + " and " + csharp_name(b.type));
        out->type = t;
        out->code = "(" + c.code + " ? " + conv(a, t) + " : " + conv(b, t) + ")";
        return true;
    }

    static int prec_of(const std::string& op) {
        if (op == "||") return 1; if (op == "&&") return 2; if (op == "|") return 3; if (op == "^") return 4; if (op == "&") return 5;
        if (op == "==" || op == "!=") return 6;
        if (op == "<" || op == ">" || op == "<=" || op == ">=") return 7;
        if (op == "<<" || op == ">>" || op == ">>>") return 8;
        if (op == "+" || op == "-") return 9;
        if (op == "*" || op == "/" || op == "%") return 10;
        return -1;
    }

    bool binary(int min_prec, Node* out) {
        Node lhs;
        if (!unary(&lhs)) return false;
        while (peek().kind == Tok::PUNCT) {
            std::string op = peek().text;
            int p = prec_of(op);
            if (p < 0 || p < min_prec) break;
            ++pos_;
            Node rhs;
            if (!binary(p + 1, &rhs)) return false;
            Node r;
            if (!apply_binary(op, lhs, rhs, &r)) return false;
            lhs = r;
        }
        *out = lhs;
        return true;
    }

    bool apply_binary(const std::string& op, const Node& a, const Node& b, Node* r) {
        if (op == "&&" || op == "||") {
            if (a.type != T_BOOL || b.type != T_BOOL) return fail("operands of " + op + " must be bool");
            r->type = T_BOOL; r->code = "(" + a.code + " " + op + " " + b.code + ")";
            return true;
        }
        if ((op == "&" || op == "|" || op == "^") && a.type == T_BOOL && b.type == T_BOOL) {
            r->type = T_BOOL; r->code = "((bool)(" + a.code + " " + op + " " + b.code + "))";
            return true;
        }
        if ((op == "==" || op == "!=") && a.type == T_BOOL && b.type == T_BOOL) {
            r->type = T_BOOL; r->code = "(" + a.code + " " + op + " " + b.code + ")";
            return true;
        }
        if (op == "<<" || op == ">>" || op == ">>>") {
            if (!is_integral(a.type) || !is_integral(b.type)) return fail("shift needs integral operands");
            int t = promote_unary(a.type);
            if (!(implicit_ok(b.type, T_I32) || (b.const_int))) return fail("shift count must convert to int");
            const char* mask = (t == T_I64 || t == T_U64) ? "63" : "31";
            std::string cnt = "(((int)(" + b.code + ")) & " + mask + ")";
            std::string ut = cuda_name(unsigned_of(t));
            r->type = t;
            if (op == "<<" || op == ">>>" )
                r->code = std::string("((") + cuda_name(t) + ")((" + ut + ")(" + conv(a, t) + ") " + (op == "<<" ? "<<" : ">>") + " " + cnt + "))";
            else
                r->code = "(" + conv(a, t) + " >> " + cnt + ")";
            return true;
        }
        int t = promote_binary(a, b);
        if (t == T_NONE) return fail(std::string("operator ") + op + " cannot be applied to " + csharp_name(a.type) + " and " + csharp_name(b.type));
        std::string ca = conv(a, t), cb = conv(b, t);
        if (op == "==" || op == "!=" || op == "<" || op == ">" || op == "<=" || op == ">=") {
            r->type = T_BOOL; r->code = "(" + ca + " " + op + " " + cb + ")";
            return true;
        }
        if (op == "&" || op == "|" || op == "^") {
            if (!is_integral(t)) return fail("operator " + op + " needs integral operands");
            r->type = t; r->code = "(" + ca + " " + op + " " + cb + ")";
            return true;
        }
        r->type = t;
        if (op == "%" && is_float(t)) {
            r->code = std::string(t == T_F32 ? "fmodf(" : "fmod(") + ca + ", " + cb + ")";
        } else if ((op == "+" || op == "-" || op == "*") && is_signed_int(t)) {
            // C# integer arithmetic wraps (unchecked context); do it in the unsigned type so C++ agrees.
            std::string ut = cuda_name(unsigned_of(t));
            r->code = std::string("((") + cuda_name(t) + ")((" + ut + ")(" + ca + ") " + op + " (" + ut + ")(" + cb + ")))";
        } else if ((op == "/" || op == "%") && is_integral(t) && !kernel_mode && !(b.const_int && b.cval != 0)) {
            // C# throws DivideByZeroException on a zero divisor and OverflowException on MinValue / -1: the helpers note
            // either in the module's fault word (the host turns it into the error) and return 0.
            // (`keep`: an element an earlier Where has dropped is never divided in C#, so it cannot fault here either)
            r->code = std::string(op == "/" ? "dcb_idiv<" : "dcb_irem<") + cuda_name(t) + ">(" + ca + ", " + cb + ", keep)";
        } else {
            r->code = "(" + ca + " " + op + " " + cb + ")";
        }
        if (a.const_int && b.const_int && t == T_I32) {   // fold int constants so narrowing rules keep working
            long long v = 0; bool ok = true;
            if (op == "+") v = a.cval + b.cval; else if (op == "-") v = a.cval - b.cval; else if (op == "*") v = a.cval * b.cval;
            else if (op == "/" && b.cval != 0) v = a.cval / b.cval; else if (op == "%" && b.cval != 0) v = a.cval % b.cval; else ok = false;
            if (ok && v >= -2147483648LL && v <= 2147483647LL) { r->const_int = true; r->cval = v; }
        }
        return true;
    }

    bool unary(Node* out) {
        if (peek().kind == Tok::PUNCT) {
            const std::string op = peek().text;
            if (op == "-" || op == "+" || op == "!" || op == "~") {
                ++pos_;
                // -2147483648 and -9223372036854775808 are int / long literals.
                if (op == "-" && peek().kind == Tok::NUM) {
                    std::string raw = peek().text; std::string digits;
                    for (char ch : raw) if (ch != '_') digits += ch;
                    if (digits == "2147483648") { ++pos_; out->type = T_I32; out->code = "(-2147483647 - 1)"; out->const_int = true; out->cval = -2147483648LL; return postfix(out); }
                    if (digits == "9223372036854775808" || digits == "9223372036854775808L" || digits == "9223372036854775808l") {
                        ++pos_; out->type = T_I64; out->code = "(-9223372036854775807LL - 1LL)"; return postfix(out);
                    }
                }
                Node a;
                if (!unary(&a)) return false;
                if (op == "!") {
                    if (a.type != T_BOOL) return fail("operand of ! must be bool");
                    out->type = T_BOOL; out->code = "(!" + a.code + ")"; return true;
                }
                if (!is_numeric(a.type)) return fail("operand of unary " + op + " must be numeric");
                int t = promote_unary(a.type);
                if (op == "~") {
                    if (!is_integral(t)) return fail("operand of ~ must be integral");
                    out->type = t; out->code = "(~" + conv(a, t) + ")"; return true;
                }
                if (op == "+") { out->type = t; out->code = conv(a, t); out->const_int = a.const_int; out->cval = a.cval; return true; }
                if (t == T_U32) t = T_I64;
                if (t == T_U64) return fail("unary minus cannot be applied to ulong");
                out->type = t;
                if (is_signed_int(t)) {
                    std::string ut = cuda_name(unsigned_of(t));
                    out->code = std::string("((") + cuda_name(t) + ")(0u - (" + ut + ")(" + conv(a, t) + ")))";
                } else {
                    out->code = "(-" + conv(a, t) + ")";
                }
                if (a.const_int) { out->const_int = true; out->cval = -a.cval; }
                return true;
            }
            // cast: '(' type ')' unary
            if (op == "(" && peek(1).kind == Tok::IDENT && type_keyword(peek(1).text) != T_NONE && is_punct(")", 2)) {
                int to = type_keyword(peek(1).text);
                pos_ += 3;
                Node a;
                if (!unary(&a)) return false;
                if (to == T_BOOL) {
                    if (a.type != T_BOOL) return fail("cannot cast to bool");
                    *out = a; return true;
                }
                if (!is_numeric(a.type)) return fail(std::string("cannot cast ") + csharp_name(a.type) + " to " + csharp_name(to));
                out->type = to; out->code = conv(a, to);
                if (a.const_int && to == T_I32) { out->const_int = true; out->cval = a.cval; }
                return true;
            }
        }
        Node p;
        if (!primary(&p)) return false;
        *out = p;
        return postfix(out);
    }

    bool postfix(Node* out) { (void)out; return true; }

    bool number(const std::string& raw, Node* out) {
        std::string s;
        for (char c : raw) if (c != '_') s += c;
        std::string body = s, suf;
        bool hex = s.size() > 2 && s[0] == '0' && (s[1] == 'x' || s[1] == 'X');
        bool bin = s.size() > 2 && s[0] == '0' && (s[1] == 'b' || s[1] == 'B');
        size_t e = s.size();
        if (hex) { while (e > 2 && (s[e - 1] == 'u' || s[e - 1] == 'U' || s[e - 1] == 'l' || s[e - 1] == 'L')) --e; }
        else { while (e > 0 && isalpha((unsigned char)s[e - 1])) --e; }   // an exponent's 'e' is always followed by digits
        body = s.substr(0, e); suf = s.substr(e);
        for (auto& ch : suf) ch = (char)tolower((unsigned char)ch);
        bool real = !hex && !bin && (body.find('.') != std::string::npos || body.find('e') != std::string::npos || body.find('E') != std::string::npos);
        if (suf == "m") return fail("decimal literals are not supported");
        if (suf == "f") { float v = strtof(body.c_str(), nullptr); out->type = T_F32; out->code = fmt_f32(v); return true; }
        if (suf == "d" || (real && suf.empty())) { double v = strtod(body.c_str(), nullptr); out->type = T_F64; out->code = fmt_f64(v); return true; }
        if (real) return fail("bad numeric suffix '" + suf + "'");
        unsigned long long v = 0;
        errno = 0;
        if (bin) v = strtoull(body.c_str() + 2, nullptr, 2); else v = strtoull(body.c_str(), nullptr, hex ? 16 : 10);
        if (errno != 0) return fail("integer literal out of range");
        bool has_u = suf.find('u') != std::string::npos, has_l = suf.find('l') != std::string::npos;
        if (!suf.empty() && !(suf == "u" || suf == "l" || suf == "ul" || suf == "lu")) return fail("bad numeric suffix '" + suf + "'");
        int t;
        if (has_u && has_l) t = T_U64;
        else if (has_u) t = v <= 0xffffffffull ? T_U32 : T_U64;
        else if (has_l) t = v <= 0x7fffffffffffffffull ? T_I64 : T_U64;
        else t = v <= 0x7fffffffull ? T_I32 : v <= 0xffffffffull ? T_U32 : v <= 0x7fffffffffffffffull ? T_I64 : T_U64;
        out->type = t;
        char buf[48];
        switch (t) {
            case T_I32: snprintf(buf, sizeof buf, "%llu", v); out->const_int = true; out->cval = (long long)v; break;
            case T_U32: snprintf(buf, sizeof buf, "%lluu", v); break;
            case T_I64: snprintf(buf, sizeof buf, "%lluLL", v); break;
            default: snprintf(buf, sizeof buf, "%lluULL", v); break;
        }
        out->code = buf;
        return true;
    }

    bool args(std::vector<Node>* out) {
        if (!expect("(")) return false;
        if (accept(")")) return true;
        while (true) {
            Node a;
            if (!ternary(&a)) return false;
            out->push_back(a);
            if (accept(")")) return true;
            if (!expect(",")) return false;
        }
    }

    bool primary(Node* out) {
        const Tok& t = peek();
        if (t.kind == Tok::NUM) { ++pos_; return number(t.text, out); }
        if (t.kind == Tok::PUNCT && t.text == "(") {
            ++pos_;
            Node a;
            if (!ternary(&a) || !expect(")")) return false;
            *out = a; out->code = a.code;
            return true;
        }
        if (t.kind != Tok::IDENT) return fail("unexpected '" + t.text + "'");
        std::string id = t.text;
        ++pos_;
        if (id == "true" || id == "false") { out->type = T_BOOL; out->code = id; return true; }
        auto it = params_.find(id);
        if (it != params_.end() && it->second.is_buffer) {
            const Node& buf = it->second;
            if (accept("[")) {
                Node idx;
                if (!ternary(&idx) || !expect("]")) return false;
                if (!is_integral(idx.type)) return fail("an index must be an integer");
                out->type = buf.type; out->is_lvalue = true;
                out->code = buf.code + "[" + idx.code + "]";
                return true;
            }
            if (is_punct(".") && peek(1).kind == Tok::IDENT && peek(1).text == "Length") {
                pos_ += 2; used_length = true;
                out->type = T_I32; out->code = "((int)__length)";
                return true;
            }
            return fail("buffer '" + id + "' can only be indexed or asked for its Length");
        }
        if (it != params_.end() && !is_punct(".")) { *out = it->second; return true; }
        if (kernel_mode && (id == "KernelContext" || id == "Kernel") && is_punct(".") && peek(1).kind == Tok::IDENT &&
            is_punct(".", 2) && peek(3).kind == Tok::IDENT) {
            const std::string what = peek(1).text, axis = peek(3).text;
            const char* intr = what == "ThreadId" ? "threadIdx" : what == "BlockId" ? "blockIdx" : what == "BlockDim" ? "blockDim" : what == "GridDim" ? "gridDim" : nullptr;
            if (intr && (axis == "X" || axis == "Y" || axis == "Z")) {
                pos_ += 4;
                const std::string a = axis == "X" ? "x" : axis == "Y" ? "y" : "z";
                if (axis == "Y") max_dim = std::max(max_dim, 2);
                if (axis == "Z") max_dim = std::max(max_dim, 3);
                out->type = T_I32;
                if (what == "ThreadId" && thread_id_is_global) out->code = "((int)(blockIdx." + a + " * blockDim." + a + " + threadIdx." + a + "))";
                else out->code = std::string("((int)") + intr + "." + a + ")";
                return true;
            }
        }
        if (id == "System" && is_punct(".")) { ++pos_; if (peek().kind != Tok::IDENT) return fail("bad qualified name"); id = peek().text; ++pos_; }
        if (is_punct(".") && peek(1).kind == Tok::IDENT) {
            std::string member = peek(1).text;
            pos_ += 2;
            if (is_punct("(")) {
                std::vector<Node> a;
                if (!args(&a)) return false;
                return call(id, member, a, out);
            }
            return static_member(id, member, out);
        }
        return fail("unknown identifier '" + id + "' (only lambda parameters, literals, Math/MathF and numeric type members are translatable)");
    }

    bool static_member(const std::string& cls, const std::string& m, Node* out) {
        int t = type_keyword(cls);
        auto set = [&](int ty, const std::string& code) { out->type = ty; out->code = code; return true; };
        if (cls == "Math") {
            if (m == "PI") return set(T_F64, "3.1415926535897931");
            if (m == "E") return set(T_F64, "2.7182818284590451");
            if (m == "Tau") return set(T_F64, "6.2831853071795862");
        } else if (cls == "MathF") {
            if (m == "PI") return set(T_F32, "3.14159274f");
            if (m == "E") return set(T_F32, "2.71828175f");
            if (m == "Tau") return set(T_F32, "6.28318548f");
        } else if (t == T_F32) {
            if (m == "MaxValue") return set(T_F32, "3.40282347e+38f");
            if (m == "MinValue") return set(T_F32, "(-3.40282347e+38f)");
            if (m == "Epsilon") return set(T_F32, "__int_as_float(1)");
            if (m == "NaN") return set(T_F32, "__int_as_float(0xffc00000)");
            if (m == "PositiveInfinity") return set(T_F32, "__int_as_float(0x7f800000)");
            if (m == "NegativeInfinity") return set(T_F32, "__int_as_float(0xff800000)");
        } else if (t == T_F64) {
            if (m == "MaxValue") return set(T_F64, "1.7976931348623157e+308");
            if (m == "MinValue") return set(T_F64, "(-1.7976931348623157e+308)");
            if (m == "Epsilon") return set(T_F64, "__longlong_as_double(1LL)");
            if (m == "NaN") return set(T_F64, "__longlong_as_double(0xfff8000000000000LL)");
            if (m == "PositiveInfinity") return set(T_F64, "__longlong_as_double(0x7ff0000000000000LL)");
            if (m == "NegativeInfinity") return set(T_F64, "__longlong_as_double(0xfff0000000000000LL)");
        } else if (is_integral(t)) {
            static const char* maxv[] = {"", "((signed char)127)", "((unsigned char)255)", "((short)32767)", "((unsigned short)65535)",
                                         "2147483647", "4294967295u", "9223372036854775807LL", "18446744073709551615ULL"};
            static const char* minv[] = {"", "((signed char)(-128))", "((unsigned char)0)", "((short)(-32768))", "((unsigned short)0)",
                                         "(-2147483647 - 1)", "0u", "(-9223372036854775807LL - 1LL)", "0ULL"};
            if (m == "MaxValue") return set(t, maxv[t]);
            if (m == "MinValue") return set(t, minv[t]);
        }
        return fail("unknown member " + cls + "." + m);
    }

    bool call(const std::string& cls, const std::string& m, std::vector<Node>& a, Node* out) {
        auto need = [&](size_t k) { return a.size() == k ? true : fail(cls + "." + m + " takes " + std::to_string(k) + " argument(s)"); };
        for (const Node& n : a) if (!is_numeric(n.type)) return fail("argument of " + cls + "." + m + " must be numeric");
        int tk = type_keyword(cls);
        if (is_float(tk) && (m == "IsNaN" || m == "IsInfinity" || m == "IsFinite" || m == "IsPositiveInfinity" || m == "IsNegativeInfinity" || m == "IsNegative")) {
            if (!need(1) || !implicit_ok(a[0].type, tk)) return fail("bad argument for " + cls + "." + m);
            std::string x = conv(a[0], tk);
            out->type = T_BOOL;
            if (m == "IsNaN") out->code = "(" + x + " != " + x + ")";
            else if (m == "IsInfinity") out->code = "(isinf(" + x + ") != 0)";
            else if (m == "IsFinite") out->code = "(isfinite(" + x + ") != 0)";
            else if (m == "IsPositiveInfinity") out->code = "(isinf(" + x + ") != 0 && " + x + " > 0)";
            else if (m == "IsNegativeInfinity") out->code = "(isinf(" + x + ") != 0 && " + x + " < 0)";
            else out->code = "(signbit(" + x + ") != 0)";
            return true;
        }
        if (cls != "Math" && cls != "MathF") return fail("calls to " + cls + "." + m + " are not translatable");
        const bool f = (cls == "MathF");
        const int ft = f ? T_F32 : T_F64;
        struct Fn { const char* cs; const char* cu; int nargs; };
        static const Fn fns[] = {
            {"Sqrt", "sqrt", 1}, {"Cbrt", "cbrt", 1}, {"Sin", "sin", 1}, {"Cos", "cos", 1}, {"Tan", "tan", 1}, {"Asin", "asin", 1},
            {"Acos", "acos", 1}, {"Atan", "atan", 1}, {"Sinh", "sinh", 1}, {"Cosh", "cosh", 1}, {"Tanh", "tanh", 1}, {"Exp", "exp", 1},
            {"Log", "log", 1}, {"Log10", "log10", 1}, {"Log2", "log2", 1}, {"Floor", "floor", 1}, {"Ceiling", "ceil", 1},
            {"Truncate", "trunc", 1}, {"Round", "rint", 1} /* C# rounds half to even */, {"Pow", "pow", 2}, {"Atan2", "atan2", 2},
            {"FusedMultiplyAdd", "fma", 3}, {"IEEERemainder", "remainder", 2}, {nullptr, nullptr, 0}};
        for (const Fn* fn = fns; fn->cs; ++fn) {
            if (m != fn->cs) continue;
            if (!need((size_t)fn->nargs)) return false;
            std::string code = std::string(fn->cu) + (f ? "f(" : "(");
            for (size_t i = 0; i < a.size(); ++i) {
                if (!implicit_ok(a[i].type, ft) && !a[i].const_int) return fail(std::string("argument of ") + cls + "." + m + " must convert to " + csharp_name(ft));
                code += (i ? ", " : "") + conv(a[i], ft);
            }
            out->type = ft; out->code = code + ")";
            return true;
        }
        if (m == "Abs") {
            if (!need(1)) return false;
            int t = a[0].type;
            if (f) { if (!implicit_ok(t, T_F32)) return fail("bad argument for MathF.Abs"); out->type = T_F32; out->code = "fabsf(" + conv(a[0], T_F32) + ")"; return true; }
            if (t == T_U8) t = T_I16; else if (t == T_U16) t = T_I32; else if (t == T_U32) t = T_I64; else if (t == T_U64) return fail("Math.Abs(ulong) is ambiguous in C#");
            out->type = t;
            std::string x = conv(a[0], t);
            if (t == T_F32) out->code = "fabsf(" + x + ")";
            else if (t == T_F64) out->code = "fabs(" + x + ")";
            else out->code = std::string("((") + cuda_name(t) + ")(" + x + " < 0 ? -" + x + " : " + x + "))";
            return true;
        }
        if (m == "Min" || m == "Max") {
            if (!need(2)) return false;
            int t = f ? T_F32 : common_type(a[0], a[1]);
            if (t == T_NONE) return fail("no common type for " + cls + "." + m);
            std::string x = conv(a[0], t), y = conv(a[1], t);
            out->type = t;
            if (is_float(t)) out->code = std::string(m == "Min" ? "dcb_net_min(" : "dcb_net_max(") + x + ", " + y + ")";
            else out->code = std::string("((") + cuda_name(t) + ")(" + x + (m == "Min" ? " < " : " > ") + y + " ? " + x + " : " + y + "))";
            return true;
        }
        if (m == "Clamp") {
            if (!need(3)) return false;
            Node ab; ab.type = f ? T_F32 : common_type(a[0], a[1]);
            int t = f ? T_F32 : (ab.type == T_NONE ? T_NONE : common_type(ab, a[2]));
            if (t == T_NONE) return fail("no common type for Clamp");
            std::string v = conv(a[0], t), lo = conv(a[1], t), hi = conv(a[2], t);
            out->type = t;
            out->code = std::string("((") + cuda_name(t) + ")(" + v + " < " + lo + " ? " + lo + " : (" + v + " > " + hi + " ? " + hi + " : " + v + ")))";
            return true;
        }
        if (m == "Sign") {
            if (!need(1)) return false;
            std::string x = a[0].code;
            out->type = T_I32; out->code = "((" + x + " > 0) - (" + x + " < 0))";
            return true;
        }
        return fail(cls + "." + m + " is not translatable");
    }
};

bool translate_lambda(const std::string& lambda, const std::vector<std::string>& args, const std::vector<int>& arg_types,
                      std::string* code, int* result_type, std::string* err) {
    std::vector<Tok> toks;
    if (!lex(lambda, &toks, err)) return false;
    // header: ident | ( [type] ident {, [type] ident} ) then =>
    size_t i = 0;
    std::vector<std::string> names;
    auto is_p = [&](size_t k, const char* p) { return k < toks.size() && toks[k].kind == Tok::PUNCT && toks[k].text == p; };
    if (toks[i].kind == Tok::IDENT) { names.push_back(toks[i].text); ++i; }
    else if (is_p(i, "(")) {
        ++i;
        while (true) {
            if (toks[i].kind != Tok::IDENT) { *err = "bad lambda parameter list"; return false; }
            if (toks[i + 1].kind == Tok::IDENT) ++i;   // explicit parameter type: skip it, the element type rules
            names.push_back(toks[i].text); ++i;
            if (is_p(i, ")")) { ++i; break; }
            if (!is_p(i, ",")) { *err = "bad lambda parameter list"; return false; }
            ++i;
        }
    } else { *err = "lambda must start with its parameter list"; return false; }
    if (!is_p(i, "=>")) { *err = "expected '=>' after the lambda parameters"; return false; }
    ++i;
    if (names.size() != args.size()) {
        *err = "lambda takes " + std::to_string(names.size()) + " parameter(s), the operator supplies " + std::to_string(args.size());
        return false;
    }
    std::map<std::string, Node> params;
    for (size_t k = 0; k < names.size(); ++k) { Node n; n.code = args[k]; n.type = arg_types[k]; params[names[k]] = n; }
    std::vector<Tok> body(toks.begin() + i, toks.end());
    Parser p(body, params);
    Node r;
    if (!p.parse(&r, err)) return false;
    *code = r.code; *result_type = r.type;
    return true;
}

// ---------------------------------------------------------------------------------------------- [Kernel] methods
namespace {

struct MethodTranslator {
    const std::vector<Tok>& t;
    std::map<std::string, Node> syms;
    Parser ex;
    std::string err;
    std::string body;

    MethodTranslator(const std::vector<Tok>& toks) : t(toks), ex(toks, syms) { ex.kernel_mode = true; }

    const Tok& peek(size_t k = 0) const { return t[std::min(ex.pos_ + k, t.size() - 1)]; }
    bool is_p(const char* p, size_t k = 0) const { return peek(k).kind == Tok::PUNCT && peek(k).text == p; }
    bool is_id(const char* p, size_t k = 0) const { return peek(k).kind == Tok::IDENT && peek(k).text == p; }
    bool accept(const char* p) { if (is_p(p)) { ++ex.pos_; return true; } return false; }
    bool fail(const std::string& m) { if (err.empty()) err = m; return false; }
    bool expect(const char* p) { return accept(p) ? true : fail(std::string("expected '") + p + "' near '" + peek().text + "'"); }
    bool expr(Node* n) { std::string e; if (!ex.parse_expr(n, &e)) return fail(e); return true; }

    static int scalar_type(const std::string& s) {
        static const std::map<std::string, int> m = {{"sbyte", T_I8}, {"byte", T_U8}, {"short", T_I16}, {"ushort", T_U16}, {"int", T_I32},
            {"uint", T_U32}, {"long", T_I64}, {"ulong", T_U64}, {"float", T_F32}, {"double", T_F64}, {"bool", T_BOOL}};
        auto it = m.find(s);
        return it == m.end() ? T_NONE : it->second;
    }

    bool assign_to(const Node& lhs, const std::string& op, const Node& rhs, std::string* out) {
        if (!lhs.is_lvalue) return fail("the left side of an assignment must be a variable or a buffer element");
        if (op == "=") {
            if (lhs.type == T_BOOL || rhs.type == T_BOOL) {
                if (lhs.type != rhs.type) return fail("cannot convert between bool and a number");
                *out = lhs.code + " = " + rhs.code; return true;
            }
            if (rhs.type != lhs.type && !implicit_ok(rhs.type, lhs.type) && !(rhs.const_int && const_fits(rhs.cval, lhs.type)))
                return fail(std::string("cannot implicitly convert ") + csharp_name(rhs.type) + " to " + csharp_name(lhs.type));
            *out = lhs.code + " = " + conv(rhs, lhs.type);
            return true;
        }
        Node r; std::string e;
        if (!ex.binop(op.substr(0, op.size() - 1), lhs, rhs, &r, &e)) return fail(e);
        *out = lhs.code + " = " + conv(r, lhs.type);   // a compound assignment casts back to the left type, as in C#
        return true;
    }

    // expression statement without the trailing ';' (also used for the init / increment parts of a for loop)
    bool simple(std::string* out) {
        if (is_p("++") || is_p("--")) {
            const std::string op = peek().text; ++ex.pos_;
            Node v; if (!expr(&v)) return false;
            Node one; one.type = T_I32; one.code = "1"; one.const_int = true; one.cval = 1;
            return assign_to(v, op == "++" ? "+=" : "-=", one, out);
        }
        Node lhs; if (!expr(&lhs)) return false;
        if (is_p("++") || is_p("--")) {
            const std::string op = peek().text; ++ex.pos_;
            Node one; one.type = T_I32; one.code = "1"; one.const_int = true; one.cval = 1;
            return assign_to(lhs, op == "++" ? "+=" : "-=", one, out);
        }
        static const char* ops[] = {"=", "+=", "-=", "*=", "/=", "%=", "&=", "|=", "^=", "<<=", ">>=", ">>>=", nullptr};
        for (int i = 0; ops[i]; ++i) {
            if (is_p(ops[i])) {
                ++ex.pos_;
                Node rhs; if (!expr(&rhs)) return false;
                return assign_to(lhs, ops[i], rhs, out);
            }
        }
        return fail("only assignments, ++ and -- can be used as statements");
    }

    bool declaration(std::string* out) {
        const std::string tname = peek().text; ++ex.pos_;
        int ty = tname == "var" ? T_NONE : scalar_type(tname);
        std::string s;
        while (true) {
            if (peek().kind != Tok::IDENT) return fail("expected a variable name");
            const std::string name = peek().text; ++ex.pos_;
            if (syms.count(name)) return fail("'" + name + "' is already defined");
            Node v; v.code = name; v.is_lvalue = true;
            if (accept("=")) {
                Node init; if (!expr(&init)) return false;
                v.type = ty == T_NONE ? init.type : ty;
                std::string a;
                if (!assign_to(v, "=", init, &a)) return false;
                s += std::string(cuda_name(v.type)) + " " + a + ";";
            } else {
                if (ty == T_NONE) return fail("a 'var' declaration needs an initialiser");
                v.type = ty;
                s += std::string(cuda_name(ty)) + " " + name + ";";
            }
            syms[name] = v;
            if (!accept(",")) break;
            s += " ";
        }
        *out = s;
        return true;
    }

    bool statement(int depth) {
        const std::string ind((size_t)depth * 4, ' ');
        if (accept("{")) {
            const std::map<std::string, Node> outer = syms;    // names declared inside the block end with it
            body += ind + "{\n";
            while (!is_p("}")) { if (peek().kind == Tok::END) return fail("missing '}'"); if (!statement(depth + 1)) return false; }
            ++ex.pos_;
            body += ind + "}\n";
            syms = outer;
            return true;
        }
        if (is_id("if")) {
            ++ex.pos_;
            Node c; if (!expect("(") || !expr(&c) || !expect(")")) return false;
            if (c.type != T_BOOL) return fail("the condition of 'if' must be bool");
            body += ind + "if (" + c.code + ")\n";
            if (!statement(is_p("{") ? depth : depth + 1)) return false;
            if (is_id("else")) {
                ++ex.pos_;
                body += ind + "else\n";
                if (!statement(is_p("{") || is_id("if") ? depth : depth + 1)) return false;
            }
            return true;
        }
        if (is_id("while")) {
            ++ex.pos_;
            Node c; if (!expect("(") || !expr(&c) || !expect(")")) return false;
            if (c.type != T_BOOL) return fail("the condition of 'while' must be bool");
            body += ind + "while (" + c.code + ")\n";
            return statement(is_p("{") ? depth : depth + 1);
        }
        if (is_id("for")) {
            ++ex.pos_;
            if (!expect("(")) return false;
            const std::map<std::string, Node> outer = syms;    // the loop variable ends with the loop
            struct Restore { std::map<std::string, Node>& s; const std::map<std::string, Node>& o; ~Restore() { s = o; } } restore{syms, outer};
            std::string init, cond, inc;
            if (!is_p(";")) {
                if (peek().kind == Tok::IDENT && (peek().text == "var" || scalar_type(peek().text) != T_NONE) && peek(1).kind == Tok::IDENT) {
                    if (!declaration(&init)) return false;
                    init.pop_back();   // drop the ';' the declaration printed
                } else if (!simple(&init)) return false;
            }
            if (!expect(";")) return false;
            if (!is_p(";")) { Node c; if (!expr(&c)) return false; if (c.type != T_BOOL) return fail("the condition of 'for' must be bool"); cond = c.code; }
            if (!expect(";")) return false;
            if (!is_p(")")) { if (!simple(&inc)) return false; }
            if (!expect(")")) return false;
            body += ind + "for (" + init + "; " + cond + "; " + inc + ")\n";
            return statement(is_p("{") ? depth : depth + 1);
        }
        if (is_id("return")) {
            ++ex.pos_;
            if (!expect(";")) return fail("a kernel returns nothing");
            body += ind + "return;\n";
            return true;
        }
        if (peek().kind == Tok::IDENT && (peek().text == "var" || scalar_type(peek().text) != T_NONE) && peek(1).kind == Tok::IDENT) {
            std::string d; if (!declaration(&d) || !expect(";")) return false;
            body += ind + d + "\n";
            return true;
        }
        std::string st; if (!simple(&st) || !expect(";")) return false;
        body += ind + st + ";\n";
        return true;
    }
};

}  // namespace

bool translate_kernel_method(const std::string& csharp, KernelMethod* out, std::string* err) {
    std::vector<Tok> toks;
    if (!lex(csharp, &toks, err)) return false;
    MethodTranslator m(toks);
    size_t& pos = m.ex.pos_;
    // [Kernel(...)] attributes, then modifiers, then `void Name(`
    while (m.is_p("[")) {
        int depth = 0;
        do { if (m.is_p("[")) ++depth; if (m.is_p("]")) --depth; if (m.peek().kind == Tok::END) { *err = "unterminated attribute"; return false; } ++pos; } while (depth > 0);
    }
    while (m.is_id("public") || m.is_id("private") || m.is_id("internal") || m.is_id("static") || m.is_id("unsafe") || m.is_id("protected")) ++pos;
    if (!m.is_id("void")) { *err = "a [Kernel] method must be 'static void'"; return false; }
    ++pos;
    if (m.peek().kind != Tok::IDENT) { *err = "expected the method name"; return false; }
    out->name = m.peek().text; ++pos;
    if (!m.expect("(")) { *err = m.err; return false; }
    std::string sig;
    while (!m.is_p(")")) {
        if (m.is_id("in") || m.is_id("ref") || m.is_id("out") || m.is_id("this")) ++pos;
        if (m.peek().kind != Tok::IDENT) { *err = "bad parameter list"; return false; }
        std::string tname = m.peek().text; ++pos;
        KernelParam kp;
        int elem = T_NONE;
        const bool generic = tname == "ReadOnlySpan" || tname == "Span" || tname == "ReadOnlyMemory" || tname == "Memory" ||
                             tname == "IUnifiedMemoryBuffer" || tname == "UnifiedBuffer";
        if (generic) {
            if (!m.expect("<") || m.peek().kind != Tok::IDENT) { *err = "bad generic parameter type"; return false; }
            elem = MethodTranslator::scalar_type(m.peek().text); ++pos;
            if (!m.expect(">")) { *err = m.err; return false; }
            kp.is_buffer = true;
            kp.is_readonly = tname == "ReadOnlySpan" || tname == "ReadOnlyMemory";
        } else {
            elem = MethodTranslator::scalar_type(tname);
            if (m.is_p("[") && m.is_p("]", 1)) { pos += 2; kp.is_buffer = true; kp.is_readonly = false; }
        }
        if (elem == T_NONE) { *err = "parameter type '" + tname + "' is not supported in a CUDA kernel"; return false; }
        if (m.peek().kind != Tok::IDENT) { *err = "expected a parameter name"; return false; }
        kp.name = m.peek().text; ++pos;
        kp.elem_type = elem;
        Node n; n.code = kp.name; n.type = elem; n.is_buffer = kp.is_buffer; n.is_lvalue = !kp.is_buffer;
        m.syms[kp.name] = n;
        if (!sig.empty()) sig += ", ";
        if (kp.is_buffer) sig += std::string(kp.is_readonly ? "const " : "") + cuda_name(elem) + "* " + kp.name;
        else sig += std::string(cuda_name(elem)) + " " + kp.name;
        out->params.push_back(kp);
        if (!m.accept(",")) break;
    }
    if (!m.expect(")")) { *err = m.err; return false; }
    // In DotCompute's CPU invoker ThreadId is the global work-item index (BlockId reads 0). A body that never names BlockId,
    // BlockDim or GridDim therefore means the global index by ThreadId; spelled with block arithmetic it is taken literally.
    bool names_blocks = false;
    for (const Tok& tk : toks) if (tk.kind == Tok::IDENT && (tk.text == "BlockId" || tk.text == "BlockDim" || tk.text == "GridDim")) names_blocks = true;
    m.ex.thread_id_is_global = !names_blocks;
    if (!m.is_p("{")) { *err = "expected the method body"; return false; }
    ++pos;
    while (!m.is_p("}")) {
        if (m.peek().kind == Tok::END) { *err = "missing '}' at the end of the method"; return false; }
        if (!m.statement(1)) { *err = m.err; return false; }
    }
    out->needs_length = m.ex.used_length;
    out->dimensions = m.ex.max_dim;
    if (out->needs_length) sig += std::string(sig.empty() ? "" : ", ") + "const unsigned int __length";
    out->cuda_source = "extern \"C\" __global__ void " + out->name + "(" + sig + ") {\n" + m.body + "}\n";
    return true;
}

// ---------------------------------------------------------------------------------------------- chains
bool build_chain(int t0, int t1, const std::vector<OpSpec>& ops, ChainInfo* info, std::string* err, int* status) {
    *status = ST_INVALID_ARGUMENT;
    if (!(t0 >= T_I8 && t0 <= T_BOOL)) { *err = "bad source element type"; return false; }
    if (ops.empty()) { *err = "a query needs a terminal operator"; return false; }
    info->in0 = t0; info->in1 = T_NONE; info->n_in = 1; info->has_filter = false;
    std::string body, key = std::string(csharp_name(t0));
    int cur = t0;
    std::string cur_var = "p0";
    int nvar = 0;
    size_t nops = ops.size();
    for (size_t i = 0; i + 1 < nops; ++i) {
        const OpSpec& op = ops[i];
        std::string code; int rt = T_NONE; std::string e;
        if (op.kind == OP_ZIP) {
            if (i != 0) { *err = "Zip must be the first operator"; *status = ST_NOT_SUPPORTED; return false; }
            if (!(t1 >= T_I8 && t1 <= T_BOOL)) { *err = "Zip needs the element type of the second sequence"; return false; }
            info->in1 = t1; info->n_in = 2;
            if (!translate_lambda(op.lambda, {"p0", "p1"}, {t0, t1}, &code, &rt, &e)) { *err = "Zip: " + e; *status = ST_NOT_SUPPORTED; return false; }
            key += std::string("|Z(") + csharp_name(t1) + "):" + code;
        } else if (op.kind == OP_SELECT) {
            if (!translate_lambda(op.lambda, {cur_var}, {cur}, &code, &rt, &e)) { *err = "Select: " + e; *status = ST_NOT_SUPPORTED; return false; }
            key += "|S:" + code;
        } else if (op.kind == OP_WHERE) {
            if (!translate_lambda(op.lambda, {cur_var}, {cur}, &code, &rt, &e)) { *err = "Where: " + e; *status = ST_NOT_SUPPORTED; return false; }
            if (rt != T_BOOL) { *err = "Where: predicate must return bool"; *status = ST_NOT_SUPPORTED; return false; }
            // Branch-free: lambdas are pure, so everything after a failed predicate may still be evaluated; the element
            // is dropped by the flag. (An early return costs a divergent branch per element inside the unrolled kernels.)
            body += "        keep = keep & " + code + ";\n";
            info->has_filter = true;
            key += "|W:" + code;
            continue;
        } else {
            *err = "only Select, Where and Zip may precede the terminal operator"; *status = ST_NOT_SUPPORTED; return false;
        }
        std::string v = "v" + std::to_string(nvar++);
        body += std::string("        const ") + cuda_name(rt) + " " + v + " = " + code + ";\n";
        cur = rt; cur_var = v;
    }
    // The canonical key names intermediate variables; make it independent of them by construction (v0, v1, ... are
    // assigned in order), so equal queries give equal keys.
    const OpSpec& term = ops.back();
    info->terminal = term.kind; info->out_type = cur; info->is_identity = (nops == 1);
    switch (term.kind) {
        case OP_TOARRAY: info->result_type = cur; info->red_mask = 0; key += "|ToArray"; break;
        case OP_COUNT: info->result_type = T_I64; info->red_mask = RED_COUNT; key += "|Count"; break;
        case OP_FIRST_INDEX: info->result_type = T_I64; info->red_mask = RED_FIRST; key += "|FirstIndex"; break;
        case OP_LAST_INDEX: info->result_type = T_I64; info->red_mask = RED_LAST; key += "|LastIndex"; break;
        case OP_MIN: case OP_MAX:
            if (!is_numeric(cur)) { *err = "Min/Max need a numeric element type"; *status = ST_NOT_SUPPORTED; return false; }
            info->result_type = cur; info->red_mask = term.kind == OP_MIN ? RED_MIN : RED_MAX; key += term.kind == OP_MIN ? "|Min" : "|Max"; break;
        case OP_SUM: case OP_AVERAGE:
            // System.Linq defines Sum and Average for int, long, float, double only.
            if (!(cur == T_I32 || cur == T_I64 || cur == T_F32 || cur == T_F64)) {
                *err = std::string("Sum/Average are defined for int, long, float and double, not ") + csharp_name(cur) + " (project with Select first)";
                *status = ST_NOT_SUPPORTED; return false;
            }
            info->red_mask = term.kind == OP_SUM ? RED_SUM : (RED_SUM | RED_COUNT);
            if (term.kind == OP_SUM) { info->result_type = cur; key += "|Sum"; info->checked_sum = (cur == T_I32 || cur == T_I64); }
            else { info->result_type = (cur == T_F32) ? T_F32 : T_F64; key += "|Average"; }
            break;
        default: *err = "the last operator must be ToArray, Sum, Min, Max, Average, Count, FirstIndex or LastIndex"; *status = ST_NOT_SUPPORTED; return false;
    }
    std::string s;
    s += "struct dcb_chain@ {\n";
    s += std::string("    typedef ") + cuda_name(t0) + " in0_t;\n";
    s += std::string("    typedef ") + cuda_name(info->n_in == 2 ? info->in1 : t0) + " in1_t;\n";
    s += std::string("    typedef ") + cuda_name(cur) + " out_t;\n";
    s += std::string("    static constexpr int n_in = ") + (info->n_in == 2 ? "2" : "1") + ";\n";
    s += std::string("    static constexpr bool has_filter = ") + (info->has_filter ? "true" : "false") + ";\n";
    s += "    static __device__ __forceinline__ bool apply(const in0_t& p0, const in1_t& p1, out_t& out) {\n";
    const bool divides = body.find("dcb_idiv<") != std::string::npos || body.find("dcb_irem<") != std::string::npos;
    if (info->has_filter) s += "        bool keep = true;\n";
    else if (divides) s += "        const bool keep = true;\n";       // the checked divisions ask whether the element is still live
    s += body;
    s += "        out = " + cur_var + std::string(";\n        return ") + (info->has_filter ? "keep" : "true") + ";\n    }\n};\n";
    info->chain_src = s;
    info->checked_div = s.find("dcb_idiv<") != std::string::npos || s.find("dcb_irem<") != std::string::npos;
    info->key = key;
    *status = 0;
    return true;
}

static std::string replace_all(std::string s, const std::string& a, const std::string& b) {
    size_t pos = 0;
    while ((pos = s.find(a, pos)) != std::string::npos) { s.replace(pos, a.size(), b); pos += b.size(); }
    return s;
}

namespace {
int pipe_bytes_per_elem(const ChainInfo& info) { return type_size(info.in0) + (info.n_in == 2 ? type_size(info.in1) : 0); }
}  // namespace

int stream_rows_for(const ChainInfo& info, int warps) {
    if (info.terminal != OP_TOARRAY || !info.has_filter) return 0;
    if (type_size(info.out_type) > type_size(info.in0)) return 0;
    // Tiles of about 20 KB (all inputs together): five slots of two resident blocks fit an SM's shared memory, and the
    // per-tile work (barriers, count descriptor, offsets) is spread over a quarter more elements than with 16 KB
    // (measured 7 % faster on float, 17 % on long). A lane keeps rows * e values in registers: at most 40.
    const int e = 16 / type_size(info.in0);
    const int cap = e <= 4 ? 10 : 8;
    const int rows = 20480 / (warps * 32 * e * pipe_bytes_per_elem(info));
    return rows < 1 ? 1 : (rows > cap ? cap : rows);
}
long long stream_tile_elems(const ChainInfo& info, int rows, int warps) { return (long long)warps * rows * 32 * (16 / type_size(info.in0)); }
long long stream_smem_bytes(const ChainInfo& info, int rows, int warps, int nbuf) {
    return (long long)nbuf * stream_tile_elems(info, rows, warps) * pipe_bytes_per_elem(info);
}
int stream_block_threads(int warps, int copy_warps) { return (warps + 2 + copy_warps) * 32; }

std::string build_program(const ChainInfo& info, const std::string& suffix, const std::string& kernels_header,
                          const Tuning& tuning, bool with_prelude) {
    const int block = tuning.block, unroll = tuning.unroll;
    std::string s;
    if (with_prelude) {
        s += "// generated by libdcb200: fused LINQ pipeline\n// key: " + info.key + "\n";
        if (kernels_header.empty()) s += "#include \"dcb_kernels.cuh\"\n"; else s += kernels_header;
        s += "\n#ifndef DCB_PRELUDE\n#define DCB_PRELUDE\n"
             "// Math.Min / Math.Max of .NET: NaN wins, and -0 orders below +0.\n"
             "template <typename T> __device__ __forceinline__ T dcb_net_min(T a, T b) {\n"
             "    if (a != b) return (a == a) ? (a < b ? a : b) : a;\n"
             "    return signbit(a) ? a : b;\n}\n"
             "template <typename T> __device__ __forceinline__ T dcb_net_max(T a, T b) {\n"
             "    if (a != b) return (a == a) ? (b < a ? a : b) : a;\n"
             "    return signbit(b) ? a : b;\n}\n"
             "// Integer division as C# defines it: a zero divisor and MinValue / -1 are errors. Bit 0 / bit 1 of the fault word.\n"
             "__device__ unsigned int dcb_fault_word = 0;\n"
             "template <typename T> __device__ __forceinline__ bool dcb_div_fault(T a, T b, bool live) {\n"
             "    if (b == T(0)) { if (live) atomicOr(&dcb_fault_word, 1u); return true; }\n"
             "    if (T(-1) < T(0) && b == T(-1) && a == T(1ull << (sizeof(T) * 8 - 1))) { if (live) atomicOr(&dcb_fault_word, 2u); return true; }\n"
             "    return false;\n}\n"
             "template <typename T> __device__ __forceinline__ T dcb_idiv(T a, T b, bool live) { return dcb_div_fault(a, b, live) ? T(0) : T(a / b); }\n"
             "template <typename T> __device__ __forceinline__ T dcb_irem(T a, T b, bool live) { return dcb_div_fault(a, b, live) ? T(0) : T(a % b); }\n"
             "#endif\n\n";
    }
    s += replace_all(info.chain_src, "@", suffix);
    const std::string C = "dcb_chain" + suffix;
    const std::string B = std::to_string(block), U = std::to_string(unroll);
    auto cast_in = [&]() { return "(const " + C + "::in0_t*)in0, (const " + C + "::in1_t*)in1"; };
    const char* variants[2] = {"vec", "scalar"};
    for (int v = 0; v < 2; ++v) {
        const std::string vec = v == 0 ? "true" : "false";
        const std::string u = v == 0 ? U : std::to_string(unroll * 2);
        if (info.terminal == OP_TOARRAY && !info.has_filter) {
            s += "extern \"C\" __global__ void __launch_bounds__(" + B + ") dcb_map_" + variants[v] + suffix +
                 "(const void* in0, const void* in1, long long n, void* out) {\n    dcb::map_body<" + C + ", " + B + ", " + u + ", " + vec + ">(" +
                 cast_in() + ", n, (" + C + "::out_t*)out);\n}\n";
        } else if (info.terminal == OP_TOARRAY) {
            const std::string CB = std::to_string(tuning.compact_block);
            const std::string rows = tuning.compact_rows > 0 ? std::to_string(tuning.compact_rows)
                                                             : "dcb::compact_rows<" + C + ", " + CB + ", " + vec + ">::value";
            const std::string bounds = tuning.compact_min_blocks > 0 ? CB + ", " + std::to_string(tuning.compact_min_blocks) : CB;
            s += "extern \"C\" __global__ void __launch_bounds__(" + bounds + ") dcb_compact_" + variants[v] + suffix +
                 "(const void* in0, const void* in1, long long n, void* out, long long out_cap, unsigned long long* desc, "
                 "unsigned int epoch, unsigned int spin_limit, long long num_tiles, const void* prev, void* res, unsigned int* abort_flag) {\n"
                 "    dcb::compact_body<" + C + ", " + CB + ", " + rows + ", " + vec + ">(" + cast_in() + ", n, (" + C +
                 "::out_t*)out, out_cap, desc, epoch, spin_limit, num_tiles, (const dcb::DeviceResult*)prev, (dcb::DeviceResult*)res, abort_flag);\n}\n";
            if (v == 0 && tuning.stream && stream_rows_for(info, tuning.stream_warps) > 0) {
                const int srow = tuning.stream_rows > 0 ? tuning.stream_rows : stream_rows_for(info, tuning.stream_warps);
                const std::string ST = std::to_string(stream_block_threads(tuning.stream_warps, tuning.stream_copy_warps));
                const std::string sbounds = tuning.stream_min_blocks > 0 ? ST + ", " + std::to_string(tuning.stream_min_blocks) : ST;
                s += "extern \"C\" __global__ void __launch_bounds__(" + sbounds + ") dcb_compact_stream" + suffix +
                     "(const void* in0, const void* in1, long long n, void* out, long long out_cap, unsigned long long* desc, "
                     "unsigned int epoch, unsigned int spin_limit, long long num_tiles, const void* prev, void* res, unsigned int* abort_flag, "
                     "unsigned int* counters, unsigned int head, unsigned int run_flags) {\n"
                     "    dcb::compact_stream_body<" + C + ", " + std::to_string(tuning.stream_warps) + ", " + std::to_string(srow) + ", " +
                     std::to_string(tuning.stream_lag) + ", " + std::to_string(tuning.stream_nbuf) + ", " + std::to_string(tuning.stream_depth) + ", " +
                     std::to_string(tuning.stream_ahead_mb) + " << 20, " + std::to_string(tuning.stream_draw_ahead) + ", " + std::to_string(tuning.stream_copy_warps) + ">(" + cast_in() + ", n, (" + C +
                     "::out_t*)out, out_cap, desc, epoch, spin_limit, num_tiles, (const dcb::DeviceResult*)prev, (dcb::DeviceResult*)res, abort_flag, counters, head, run_flags);\n}\n";
            }
        } else {
            // Keep the register count where 6 (one input) or 4 (Zip) blocks share an SM: measured as fast as 8 blocks, and
            // unlike a cap of 32 registers it leaves the once-per-launch tail (the fold of the block partials) free of spills.
            // (the ordered integer Sum keeps a lane's run of outputs in registers: 4 blocks, 64 registers)
            const std::string rb = B + ", " + std::to_string(tuning.reduce_min_blocks > 0 ? tuning.reduce_min_blocks : ((info.n_in == 2 || info.checked_sum) ? 4 : 6));
            // Sum over int / long is checked element by element in source order: its own, ordered kernel (same launch).
            const std::string body = info.checked_sum ? "dcb::sum_checked_body<" + C + ", " + B + ", " + u + ", " + vec + ">"
                                                      : "dcb::reduce_body<" + C + ", " + std::to_string(info.red_mask) + ", " + B + ", " + u + ", " + vec + ">";
            s += "extern \"C\" __global__ void __launch_bounds__(" + rb + ") dcb_reduce_" + variants[v] + suffix +
                 "(const void* in0, const void* in1, long long n, void* partials, unsigned int* ticket, void* res) {\n"
                 "    " + body + "(" + cast_in() + ", n, (dcb::Partial*)partials, ticket, (dcb::DeviceResult*)res);\n}\n";
        }
    }
    return s;
}

}  // namespace dcbt
