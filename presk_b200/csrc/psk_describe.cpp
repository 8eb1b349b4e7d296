// psk_describe: from the reference's kernel text to a launch of this executor.
//
// The reference hands an executor a `Kernel` (crates/presk-kernel/src/ir.rs:300-322): buffers and a loop nest
// over scalar operations. Its `Display` (ir.rs:495-596) prints that as text,
//
//   kernel NAME (%0 : T[ax: n, m], %1 : T[..], ..) -> %N : T[..] [arith F product F accum F [store F]] {
//     for iV in 0..BOUND { .. }     sV = EXPR     nV = EXPR     iV = EXPR     vV = EXPR
//     %B[ix, ..] = EXPR             %B[ix, ..] <v= EXPR        if COND { .. }
//   }
//
// which is the form a shim on the reference's side can produce without knowing anything of this library
// (`k.to_string()` inside `KernelExec::run`, crates/presk-kernel/src/host.rs:30). This file reads that text and
// recognises which family of the lowering table (crates/presk-kernel/src/lower.rs) the nest is: the iteration
// space, how each buffer is indexed in it (as element strides), and the steps of an elementwise group. What it
// has no family for is refused with PSK_E7005 and a message; nothing is ever approximated.
//
// Recognition goes by the nest's structure wherever the structure decides the arithmetic:
//   * a perfect nest with one store             -> PSK_OP_FUSED (lower.rs:309-372) or PSK_OP_COPY (a bare load);
//   * sums kept in a scalar or in the output    -> PSK_OP_CONTRACT (lower.rs:384-636, the row-wise `dot` of
//     lower.rs:1184) or PSK_OP_REDUCE (lower.rs:1221-1255), the summed loops in their nesting order;
// and by the kernel's name plus its buffers where the name fixes the function and every layout of it is
// bit-identical by the reference's own contract (crates/presk-kernel/src/layout.rs:6-11):
//   * `dot` in a tiled or laned form (vector statements), `softmax axis A [where]` (lower.rs:1274-1419),
//     `cross_entropy` (:1459), `embed` (:1421), `argmax` (:1490).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../../include/presk_cuda.h"

namespace {

struct Refuse {
    int code;
    std::string msg;
};
[[noreturn]] void refuse(int code, const std::string &m) { throw Refuse{code, m}; }

// ---- the tree --------------------------------------------------------------------------------------------------
struct Expr;
typedef std::shared_ptr<Expr> E;
struct Expr {
    enum Kind { Num, Load, Var, Bin, Un, Cmp, Select, ToF, ToI, Splat } kind = Num;
    std::string text;     // Num: the literal; Var: "i3", "s0", "n1", "v2"; Bin/Cmp: the operator; Un: the function
    double num = 0;
    int buf = -1;         // Load
    bool vec = false;     // a `<v>` load or operation
    std::vector<E> kids;  // Load: the indices; Bin, Cmp: two; Un, ToF, ToI, Splat: one; Select: three
};

struct Stmt {
    enum Kind { For, Set, Store, If } kind = Set;
    std::string var;      // For: the loop variable; Set: the variable assigned (i, s, n or v)
    int64_t bound = 0;    // For
    int buf = -1;         // Store
    bool vec = false;     // VStore
    std::vector<E> index; // Store
    E value;              // Set, Store; If: the condition
    std::vector<Stmt> body;
};

struct Buf {
    std::string type;     // "f32", "bf16", "i64", "int8"
    int quant_over = -1, quant_end = -1;
    std::vector<int64_t> dims;
    std::vector<std::string> names;
    int64_t numel() const { int64_t n = 1; for (auto d : dims) n *= d; return n; }
    std::vector<int64_t> strides() const
    {
        std::vector<int64_t> s(dims.size(), 1);
        for (int i = (int)dims.size() - 2; i >= 0; --i) s[i] = s[i + 1] * dims[i + 1];
        return s;
    }
};

struct Kernel {
    std::string name;
    std::vector<Buf> inputs;
    Buf output;
    bool formats = false; // an `arith .. product .. accum ..` clause: the kernel interpreter's to emulate
    std::vector<Stmt> body;
};

std::string show(const E &e)
{
    switch (e->kind) {
    case Expr::Num: return e->text;
    case Expr::Var: return e->text;
    case Expr::Load: {
        std::string s = "%" + std::to_string(e->buf) + "[";
        for (size_t i = 0; i < e->kids.size(); ++i) s += (i ? ", " : "") + show(e->kids[i]);
        return s + "]" + (e->vec ? "<v>" : "");
    }
    case Expr::Bin: case Expr::Cmp: return "(" + show(e->kids[0]) + " " + e->text + " " + show(e->kids[1]) + ")" + (e->vec ? "<v>" : "");
    case Expr::Un: return e->text + "(" + show(e->kids[0]) + ")";
    case Expr::Select: return "select(" + show(e->kids[0]) + ", " + show(e->kids[1]) + ", " + show(e->kids[2]) + ")";
    case Expr::ToF: return "real(" + show(e->kids[0]) + ")";
    case Expr::ToI: return "int(" + show(e->kids[0]) + ")";
    case Expr::Splat: return "splat(" + show(e->kids[0]) + ")";
    }
    return "?";
}

// ---- the reader ------------------------------------------------------------------------------------------------
struct Reader {
    const char *p;
    explicit Reader(const char *s) : p(s) {}
    void ws() { while (*p == ' ' || *p == '\t') ++p; }
    bool eat(const char *lit)
    {
        ws();
        size_t n = strlen(lit);
        if (strncmp(p, lit, n) == 0) { p += n; return true; }
        return false;
    }
    void want(const char *lit) { if (!eat(lit)) refuse(PSK_E7001, std::string("kernel text: `") + lit + "` was expected at `" + std::string(p, strnlen(p, 24)) + "`"); }
    int64_t integer()
    {
        ws();
        char *end;
        long long v = strtoll(p, &end, 10);
        if (end == p) refuse(PSK_E7001, std::string("kernel text: a number was expected at `") + std::string(p, strnlen(p, 24)) + "`");
        p = end;
        return v;
    }
    static bool ident_char(char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '_'; }

    E expr()
    {
        ws();
        auto e = std::make_shared<Expr>();
        if (*p == '(') {
            ++p;
            E a = expr();
            ws();
            std::string op;
            while (*p == '+' || *p == '-' || *p == '*' || *p == '/' || *p == '<' || *p == '>' || *p == '=') op.push_back(*p++);
            if (op.empty()) refuse(PSK_E7001, std::string("kernel text: an operator was expected at `") + std::string(p, strnlen(p, 24)) + "`");
            E b = expr();
            want(")");
            e->kind = (op == "+" || op == "-" || op == "*" || op == "/") ? Expr::Bin : Expr::Cmp;
            e->text = op;
            e->kids = {a, b};
            if (strncmp(p, "<v>", 3) == 0) { p += 3; e->vec = true; }
            return e;
        }
        if (*p == '%') {
            ++p;
            e->kind = Expr::Load;
            e->buf = (int)integer();
            want("[");
            ws();
            if (*p != ']') {
                for (;;) {
                    e->kids.push_back(expr());
                    if (eat(",")) continue;
                    break;
                }
            }
            want("]");
            if (strncmp(p, "<v>", 3) == 0) { p += 3; e->vec = true; }
            return e;
        }
        if ((*p >= '0' && *p <= '9') || *p == '-' || *p == '.') {
            char *end;
            e->kind = Expr::Num;
            e->num = strtod(p, &end);
            e->text.assign(p, end - p);
            p = end;
            return e;
        }
        // a word: a function, a variable, or one of Rust's spellings of a non-finite literal
        const char *q = p;
        while (ident_char(*q)) ++q;
        std::string word(p, q - p);
        if (word.empty()) refuse(PSK_E7001, std::string("kernel text: an expression was expected at `") + std::string(p, strnlen(p, 24)) + "`");
        p = q;
        if (*p == '(') {
            ++p;
            if (word == "select") {
                E c = expr(); want(","); E a = expr(); want(","); E b = expr(); want(")");
                e->kind = Expr::Select; e->kids = {c, a, b};
                return e;
            }
            E a = expr();
            want(")");
            e->kids = {a};
            if (word == "real") e->kind = Expr::ToF;
            else if (word == "int") e->kind = Expr::ToI;
            else if (word == "splat") e->kind = Expr::Splat;
            else { e->kind = Expr::Un; e->text = word; }
            return e;
        }
        if (word == "inf" || word == "NaN") {
            e->kind = Expr::Num; e->text = word; e->num = word == "inf" ? INFINITY : NAN;
            return e;
        }
        e->kind = Expr::Var;
        e->text = word;
        return e;
    }
};

std::vector<std::string> split_lines(const std::string &t)
{
    std::vector<std::string> out;
    size_t a = 0;
    while (a <= t.size()) {
        size_t b = t.find('\n', a);
        if (b == std::string::npos) b = t.size();
        out.push_back(t.substr(a, b - a));
        a = b + 1;
    }
    return out;
}

std::string trim(const std::string &s)
{
    size_t a = s.find_first_not_of(" \t\r"), b = s.find_last_not_of(" \t\r");
    return a == std::string::npos ? "" : s.substr(a, b - a + 1);
}

Buf read_spec(const std::string &text)
{
    // T[ax: n, m] with T one of f64 f32 bf16 f16 e8m15 i64 intB/OVER intB/OVER..END
    Buf b;
    size_t br = text.find('[');
    if (br == std::string::npos || text.back() != ']') refuse(PSK_E7001, "kernel text: a buffer's type `" + text + "` has no axes");
    std::string t = trim(text.substr(0, br));
    size_t slash = t.find('/');
    if (t.compare(0, 3, "int") == 0 && slash != std::string::npos) {
        b.type = t.substr(0, slash);
        std::string rest = t.substr(slash + 1);
        size_t dots = rest.find("..");
        b.quant_over = atoi(rest.c_str());
        b.quant_end = dots == std::string::npos ? b.quant_over + 1 : atoi(rest.c_str() + dots + 2);
    } else {
        b.type = t;
    }
    std::string axes = text.substr(br + 1, text.size() - br - 2);
    size_t a = 0;
    while (a < axes.size()) {
        size_t c = axes.find(',', a);
        if (c == std::string::npos) c = axes.size();
        std::string ax = trim(axes.substr(a, c - a));
        if (!ax.empty()) {
            size_t colon = ax.rfind(':');
            if (colon == std::string::npos) { b.names.push_back(""); b.dims.push_back(atoll(ax.c_str())); }
            else { b.names.push_back(trim(ax.substr(0, colon))); b.dims.push_back(atoll(ax.c_str() + colon + 1)); }
        }
        a = c + 1;
    }
    return b;
}

// One `%k : T[..]` list, split at the commas that are outside brackets.
std::vector<std::string> split_top(const std::string &s)
{
    std::vector<std::string> out;
    int depth = 0;
    size_t a = 0;
    for (size_t i = 0; i <= s.size(); ++i) {
        if (i == s.size() || (s[i] == ',' && depth == 0)) {
            std::string part = trim(s.substr(a, i - a));
            if (!part.empty()) out.push_back(part);
            a = i + 1;
        } else if (s[i] == '[') ++depth;
        else if (s[i] == ']') --depth;
    }
    return out;
}

std::vector<Stmt> read_block(const std::vector<std::string> &lines, size_t &at)
{
    std::vector<Stmt> out;
    for (; at < lines.size(); ++at) {
        std::string l = trim(lines[at]);
        if (l.empty()) continue;
        if (l == "}") return out;
        Stmt s;
        if (l.compare(0, 4, "for ") == 0) {
            // for iV in 0..BOUND {
            Reader r(l.c_str() + 4);
            r.ws();
            const char *q = r.p;
            while (Reader::ident_char(*q)) ++q;
            s.kind = Stmt::For;
            s.var.assign(r.p, q - r.p);
            r.p = q;
            r.want("in");
            r.want("0..");
            s.bound = r.integer();
            r.want("{");
            ++at;
            s.body = read_block(lines, at);
            if (at >= lines.size()) refuse(PSK_E7001, "kernel text: a `for` is not closed");
        } else if (l.compare(0, 3, "if ") == 0) {
            Reader r(l.c_str() + 3);
            s.kind = Stmt::If;
            s.value = r.expr();
            r.want("{");
            ++at;
            s.body = read_block(lines, at);
            if (at >= lines.size()) refuse(PSK_E7001, "kernel text: an `if` is not closed");
        } else if (l[0] == '%') {
            Reader r(l.c_str() + 1);
            s.kind = Stmt::Store;
            s.buf = (int)r.integer();
            r.want("[");
            r.ws();
            if (*r.p != ']') {
                for (;;) {
                    s.index.push_back(r.expr());
                    if (r.eat(",")) continue;
                    break;
                }
            }
            r.want("]");
            if (r.eat("<v=")) s.vec = true;
            else r.want("=");
            s.value = r.expr();
        } else {
            Reader r(l.c_str());
            const char *q = r.p;
            while (Reader::ident_char(*q)) ++q;
            s.kind = Stmt::Set;
            s.var.assign(r.p, q - r.p);
            r.p = q;
            r.want("=");
            s.value = r.expr();
        }
        out.push_back(std::move(s));
    }
    return out;
}

// Reads the first kernel of `text`; `*rest` is left after it.
Kernel read_kernel(const char *text, const char **rest)
{
    std::string all(text);
    size_t start = all.find("kernel ");
    if (start == std::string::npos) refuse(PSK_E7001, "kernel text: no `kernel` in it");
    size_t eol = all.find('\n', start);
    if (eol == std::string::npos) refuse(PSK_E7001, "kernel text: the header has no body");
    std::string head = all.substr(start + 7, eol - start - 7);
    Kernel k;
    // NAME (inputs) -> %N : SPEC [formats] {   -- the name may hold brackets, commas and colons, never " -> %"
    size_t arrow = head.rfind(") -> %");
    if (arrow == std::string::npos || trim(head).back() != '{') refuse(PSK_E7001, "kernel text: the header is not `NAME (..) -> %N : T[..] {`");
    size_t open = head.find(" (%0 :");
    if (open == std::string::npos || open > arrow) open = head.rfind(" (", arrow);
    if (open == std::string::npos) refuse(PSK_E7001, "kernel text: the header's inputs are missing");
    k.name = trim(head.substr(0, open));
    for (auto &part : split_top(head.substr(open + 2, arrow - open - 2))) {
        size_t colon = part.find(" : ");
        if (part[0] != '%' || colon == std::string::npos) refuse(PSK_E7001, "kernel text: an input is not `%k : T[..]`: `" + part + "`");
        if (atoi(part.c_str() + 1) != (int)k.inputs.size()) refuse(PSK_E7001, "kernel text: the inputs are not numbered in order");
        k.inputs.push_back(read_spec(trim(part.substr(colon + 3))));
    }
    std::string tail = trim(head.substr(arrow + 6)); // N : SPEC [formats] {
    tail = trim(tail.substr(0, tail.size() - 1));
    size_t colon = tail.find(" : ");
    if (colon == std::string::npos || atoi(tail.c_str()) != (int)k.inputs.size()) refuse(PSK_E7001, "kernel text: the output is not `%N : T[..]` with N the number of inputs");
    std::string ospec = tail.substr(colon + 3);
    size_t close = ospec.find(']');
    if (close == std::string::npos) refuse(PSK_E7001, "kernel text: the output's type has no axes");
    k.formats = !trim(ospec.substr(close + 1)).empty();
    k.output = read_spec(ospec.substr(0, close + 1));
    std::vector<std::string> lines = split_lines(all.substr(eol + 1));
    size_t at = 0;
    k.body = read_block(lines, at);
    if (at >= lines.size()) refuse(PSK_E7001, "kernel text: the kernel `" + k.name + "` is not closed");
    if (rest) {
        // the text after the closing line
        size_t pos = eol + 1;
        for (size_t i = 0; i <= at; ++i) pos += lines[i].size() + 1;
        *rest = text + std::min(pos, all.size());
    }
    return k;
}

// ---- from a nest to a launch -----------------------------------------------------------------------------------
int dtype_of(const std::string &t)
{
    if (t == "f64") return PSK_F64;
    if (t == "f32") return PSK_F32;
    if (t == "bf16") return PSK_BF16;
    if (t == "f16") return PSK_F16;
    if (t == "e8m15") return PSK_E8M15;
    if (t == "i64") return PSK_I64;
    if (t == "int8") return PSK_I8;
    if (t == "e4m3fn" || t == "e4m3") return PSK_E4M3;
    return -1;
}

struct Ctx {
    const Kernel &k;
    psk_launch &l;
    std::map<std::string, int> pos; // loop variable -> its axis of the iteration space
    std::map<std::string, E> scalars; // scalar variables that stand for a load (s0 = %0[i0, i1])
    int naxes = 0;
    std::vector<bool> operand_set;

    Ctx(const Kernel &kk, psk_launch &ll) : k(kk), l(ll), operand_set(PSK_MAX_INPUTS, false) {}

    const Buf &buf(int b) const { return b == (int)k.inputs.size() ? k.output : k.inputs[b]; }

    // One index of a load or store as (loop variable or "", constant): iV, (iV + c), c.
    void affine(const E &e, std::string &var, int64_t &c) const
    {
        var.clear();
        c = 0;
        if (e->kind == Expr::Var && e->text[0] == 'i') { var = e->text; return; }
        if (e->kind == Expr::Num) { c = (int64_t)e->num; return; }
        if (e->kind == Expr::Bin && e->text == "+") {
            const E &a = e->kids[0], &b = e->kids[1];
            if (a->kind == Expr::Var && a->text[0] == 'i' && b->kind == Expr::Num) { var = a->text; c = (int64_t)b->num; return; }
            if (b->kind == Expr::Var && b->text[0] == 'i' && a->kind == Expr::Num) { var = b->text; c = (int64_t)a->num; return; }
        }
        refuse(PSK_E7005, k.name + ": the index `" + show(e) + "` is not a loop variable plus a constant; this executor has no launch for such a nest");
    }

    // The element strides of a buffer over the iteration space, from the indices a load or store gives it.
    void strides_of(int b, const std::vector<E> &index, int64_t *stride, int64_t *sstride, int64_t &offset) const
    {
        const Buf &s = buf(b);
        if (index.size() != s.dims.size()) refuse(PSK_E7001, k.name + ": %" + std::to_string(b) + " has " + std::to_string(s.dims.size()) + " axes and is indexed by " + std::to_string(index.size()));
        for (int a = 0; a < PSK_MAX_AXES; ++a) { stride[a] = 0; if (sstride) sstride[a] = 0; }
        offset = 0;
        auto st = s.strides();
        std::vector<int64_t> ss(s.dims.size(), 0);
        if (s.quant_over >= 0) {
            int64_t acc = 1;
            for (int a = (int)s.dims.size() - 1; a >= 0; --a)
                if (a < s.quant_over || a >= s.quant_end) { ss[a] = acc; acc *= s.dims[a]; }
        }
        for (size_t i = 0; i < index.size(); ++i) {
            std::string var;
            int64_t c;
            affine(index[i], var, c);
            offset += c * st[i];
            if (c != 0 && s.quant_over >= 0) refuse(PSK_E7005, k.name + ": integer weights read at an offset");
            if (var.empty()) continue;
            auto it = pos.find(var);
            if (it == pos.end()) refuse(PSK_E7005, k.name + ": the index `" + var + "` of %" + std::to_string(b) + " is not a loop of the nest's iteration space");
            stride[it->second] += st[i];
            if (sstride) sstride[it->second] += ss[i];
        }
    }

    void set_operand(psk_operand &o, int b, const std::vector<E> &index)
    {
        const Buf &s = buf(b);
        memset(&o, 0, sizeof o);
        int d = dtype_of(s.type);
        if (d < 0) refuse(PSK_E7005, k.name + ": a buffer of type `" + s.type + "` is not one this executor stores");
        o.dtype = d;
        o.is_index = d == PSK_I64 ? 1 : 0;
        o.numel = s.numel();
        strides_of(b, index, o.stride, o.scale_stride, o.offset);
    }

    // Input `b` read at `index`: every load of one buffer in a nest must agree (a launch has one view an input).
    void use_input(int b, const std::vector<E> &index)
    {
        if (b < 0 || b >= (int)k.inputs.size()) refuse(PSK_E7001, k.name + ": a load of %" + std::to_string(b) + ", which is no input");
        if (b >= PSK_MAX_INPUTS) refuse(PSK_E7005, k.name + ": more inputs than a launch holds");
        psk_operand o;
        set_operand(o, b, index);
        if (operand_set[b]) {
            if (memcmp(&o, &l.in[b], sizeof o) != 0) refuse(PSK_E7005, k.name + ": %" + std::to_string(b) + " is read through two different indexings");
            return;
        }
        l.in[b] = o;
        operand_set[b] = true;
    }
};

bool is_num(const E &e, double v) { return e->kind == Expr::Num && e->num == v; }
bool same(const E &a, const E &b) { return show(a) == show(b); }
bool is_bin(const E &e, const char *op) { return e->kind == Expr::Bin && e->text == op && !e->vec; }
bool is_cmp(const E &e, const char *op) { return e->kind == Expr::Cmp && e->text == op; }
bool is_un(const E &e, const char *fn) { return e->kind == Expr::Un && e->text == fn; }

// The steps of an elementwise value (lower.rs:184-226 printed by ir.rs:509-560), innermost first. Returns the
// source of the value: an input (>= 0) or a step (-1 - k).
struct Steps {
    Ctx &c;
    std::map<std::string, int> memo;
    explicit Steps(Ctx &cc) : c(cc) {}

    int push(int prim, int nargs, int a, int b, int imm = 0)
    {
        if (c.l.n_steps >= PSK_MAX_STEPS) refuse(PSK_E7005, c.k.name + ": a group of more steps than a launch holds");
        psk_step &s = c.l.steps[c.l.n_steps];
        s.prim = prim; s.nargs = nargs; s.src[0] = a; s.src[1] = nargs == 2 ? b : 0; s.imm = imm;
        return -1 - c.l.n_steps++;
    }

    int value(const E &e0)
    {
        E e = e0;
        if (e->kind == Expr::Var && e->text[0] == 's') {
            auto it = c.scalars.find(e->text);
            if (it == c.scalars.end()) refuse(PSK_E7005, c.k.name + ": the scalar `" + e->text + "` is not a loaded value");
            e = it->second;
        }
        const std::string key = show(e);
        auto hit = memo.find(key);
        if (hit != memo.end()) return hit->second;
        int r = build(e);
        memo[key] = r;
        return r;
    }

    int build(const E &e)
    {
        const double SQRT2 = 1.4142135623730951, SQRT2PI = 2.5066282746310002;
        switch (e->kind) {
        case Expr::Load:
            if (e->vec) refuse(PSK_E7005, c.k.name + ": a vector load outside a nest this executor knows by name");
            if (dtype_of(c.buf(e->buf).type) == PSK_I64) refuse(PSK_E7005, c.k.name + ": an index read as a real without `real(..)`");
            c.use_input(e->buf, e->kids);
            return e->buf;
        case Expr::ToF: {
            const E &x = e->kids[0];
            if (x->kind != Expr::Load || dtype_of(c.buf(x->buf).type) != PSK_I64) refuse(PSK_E7005, c.k.name + ": `real` of something that is not a loaded index: " + show(e));
            c.use_input(x->buf, x->kids);
            return push(PSK_REAL, 1, x->buf, 0);
        }
        case Expr::Un: {
            static const std::pair<const char *, int> un[] = {{"neg", PSK_NEG}, {"exp", PSK_EXP}, {"log", PSK_LOG}, {"tanh", PSK_TANH}, {"sqrt", PSK_SQRT}, {"sin", PSK_SIN}, {"cos", PSK_COS}, {"abs", PSK_ABS}};
            for (auto &u : un)
                if (e->text == u.first) return push(u.second, 1, value(e->kids[0]), 0);
            refuse(PSK_E7005, c.k.name + ": `" + e->text + "` by itself is no step of a group (erf occurs inside gelu only)");
        }
        case Expr::Select: {
            const E &cnd = e->kids[0], &a = e->kids[1], &b = e->kids[2];
            // relu = select((x < 0), 0, x); heaviside = select((x > 0), 1, 0); sign = select((x < 0), -1, select((x > 0), 1, 0))
            if (is_cmp(cnd, "<") && is_num(cnd->kids[1], 0.0) && is_num(a, 0.0) && same(b, cnd->kids[0])) return push(PSK_RELU, 1, value(b), 0);
            if (is_cmp(cnd, ">") && is_num(cnd->kids[1], 0.0) && is_num(a, 1.0) && is_num(b, 0.0)) return push(PSK_HEAVISIDE, 1, value(cnd->kids[0]), 0);
            if (is_cmp(cnd, "<") && is_num(cnd->kids[1], 0.0) && is_num(a, -1.0) && b->kind == Expr::Select && is_cmp(b->kids[0], ">") && same(b->kids[0]->kids[0], cnd->kids[0]) && is_num(b->kids[0]->kids[1], 0.0) && is_num(b->kids[1], 1.0) && is_num(b->kids[2], 0.0))
                return push(PSK_SIGN, 1, value(cnd->kids[0]), 0);
            // max = select((x > y), x, y); min = select((x < y), x, y): the second operand at a tie
            if ((is_cmp(cnd, ">") || is_cmp(cnd, "<")) && same(a, cnd->kids[0]) && same(b, cnd->kids[1])) {
                const int x = value(a), y = value(b);
                return push(is_cmp(cnd, ">") ? PSK_MAX : PSK_MIN, 2, x, y);
            }
            refuse(PSK_E7005, c.k.name + ": a selection that is none of relu, heaviside, sign, max, min: " + show(e));
        }
        case Expr::Bin: {
            if (e->vec) refuse(PSK_E7005, c.k.name + ": a vector operation outside a nest this executor knows by name");
            const E &a = e->kids[0], &b = e->kids[1];
            // sigmoid = (1 / (1 + exp(neg(x))))
            if (is_bin(e, "/") && is_num(a, 1.0) && is_bin(b, "+") && is_num(b->kids[0], 1.0) && is_un(b->kids[1], "exp") && is_un(b->kids[1]->kids[0], "neg"))
                return push(PSK_SIGMOID, 1, value(b->kids[1]->kids[0]->kids[0]), 0);
            // phi(x) = ((1 + erf((x / sqrt 2))) / 2)
            auto phi_of = [&](const E &p) -> E {
                if (is_bin(p, "/") && is_num(p->kids[1], 2.0) && is_bin(p->kids[0], "+") && is_num(p->kids[0]->kids[0], 1.0) && is_un(p->kids[0]->kids[1], "erf")) {
                    const E &arg = p->kids[0]->kids[1]->kids[0];
                    if (is_bin(arg, "/") && is_num(arg->kids[1], SQRT2)) return arg->kids[0];
                }
                return nullptr;
            };
            // gelu = (x * phi(x))
            if (is_bin(e, "*")) {
                E x = phi_of(b);
                if (x && same(x, a)) return push(PSK_GELU, 1, value(a), 0);
            }
            // gelu_deriv = (phi(x) + (x * (exp((neg((x * x)) / 2)) / sqrt(2 pi))))
            if (is_bin(e, "+")) {
                E x = phi_of(a);
                if (x && is_bin(b, "*") && same(b->kids[0], x) && is_bin(b->kids[1], "/") && is_num(b->kids[1]->kids[1], SQRT2PI) && is_un(b->kids[1]->kids[0], "exp"))
                    return push(PSK_GELU_DERIV, 1, value(x), 0);
            }
            // x / n with a literal n: the cotangent of a mean (lower.rs:1257-1270)
            if (is_bin(e, "/") && b->kind == Expr::Num && b->num == std::floor(b->num) && std::fabs(b->num) < 2147483648.0 && b->num != 0.0)
                return push(PSK_DIV_N, 1, value(a), 0, (int)b->num);
            if (a->kind == Expr::Num || b->kind == Expr::Num) refuse(PSK_E7005, c.k.name + ": a literal operand has no step in a group: " + show(e));
            const int x = value(a), y = value(b);
            return push(e->text == "+" ? PSK_ADD : e->text == "-" ? PSK_SUB : e->text == "*" ? PSK_MUL : PSK_DIV, 2, x, y);
        }
        default:
            refuse(PSK_E7005, c.k.name + ": no step of a group computes `" + show(e) + "`");
        }
    }
};

void set_dims_from_output(Ctx &c)
{
    const Buf &o = c.k.output;
    if (o.dims.size() > PSK_MAX_RANK) refuse(PSK_E7005, c.k.name + ": more output axes than a launch holds");
    c.l.n_outer = (int)o.dims.size();
    for (size_t a = 0; a < o.dims.size(); ++a) c.l.dims[a] = o.dims[a];
    c.naxes = c.l.n_outer;
}

bool has_vector(const std::vector<Stmt> &b)
{
    std::vector<const Expr *> stack;
    auto scan = [&](const E &e, auto &&self) -> bool {
        if (!e) return false;
        if (e->vec || e->kind == Expr::Splat || (e->kind == Expr::Var && e->text[0] == 'v')) return true;
        for (auto &k : e->kids) if (self(k, self)) return true;
        return false;
    };
    for (auto &s : b) {
        if (s.vec || (s.kind == Stmt::Set && (s.var[0] == 'v' || s.var[0] == 'i'))) return true;
        if (scan(s.value, scan)) return true;
        for (auto &i : s.index) if (scan(i, scan)) return true;
        if (has_vector(s.body)) return true;
    }
    return false;
}

// Row-major indices of a whole buffer over consecutive axes of the space starting at `first`.
std::vector<E> iv_list(const std::vector<std::string> &vars)
{
    std::vector<E> out;
    for (auto &v : vars) {
        auto e = std::make_shared<Expr>();
        e->kind = Expr::Var;
        e->text = v;
        out.push_back(e);
    }
    return out;
}

// -- a perfect nest around one store: an elementwise group, or a copy ---------------------------------------------
bool try_elementwise(Ctx &c)
{
    const std::vector<Stmt> *body = &c.k.body;
    std::vector<std::string> vars;
    std::vector<int64_t> bounds;
    while (body->size() == 1 && (*body)[0].kind == Stmt::For) {
        vars.push_back((*body)[0].var);
        bounds.push_back((*body)[0].bound);
        body = &(*body)[0].body;
    }
    if (body->size() != 1 || (*body)[0].kind != Stmt::Store || (*body)[0].vec) return false;
    const Stmt &st = (*body)[0];
    const int out = (int)c.k.inputs.size();
    if (st.buf != out) return false;
    if (vars.size() != c.k.output.dims.size() || st.index.size() != vars.size()) return false;
    set_dims_from_output(c);
    for (size_t a = 0; a < vars.size(); ++a) {
        // the store walks the output's axes by the loops in order (lower.rs `nest` + `ivs`)
        if (!(st.index[a]->kind == Expr::Var && st.index[a]->text == vars[a]) || bounds[a] != c.k.output.dims[a]) return false;
        c.pos[vars[a]] = (int)a;
    }
    c.set_operand(c.l.out, out, st.index);
    // a bare load: a copy (slice, index, broadcast_like, split and merge of heads: lower.rs:1554-1667)
    if (st.value->kind == Expr::Load && !st.value->vec && dtype_of(c.buf(st.value->buf).type) != PSK_I64 && c.k.inputs.size() == 1) {
        c.use_input(st.value->buf, st.value->kids);
        c.l.op = PSK_OP_COPY;
        return true;
    }
    Steps steps(c);
    const int last = steps.value(st.value);
    if (last >= 0) refuse(PSK_E7005, c.k.name + ": the group's value is an input itself");
    if (last != -c.l.n_steps) refuse(PSK_E7005, c.k.name + ": the stored value is not the group's last step");
    c.l.op = PSK_OP_FUSED;
    for (size_t b = 0; b < c.k.inputs.size(); ++b)
        if (!c.operand_set[b]) refuse(PSK_E7005, c.k.name + ": input %" + std::to_string(b) + " is never read; a launch's inputs are the ones its steps name");
    return true;
}

// -- sums: a scalar or the output accumulates terms over the loops that do not index the output ------------------
struct SumNest {
    std::vector<std::pair<std::string, int64_t>> loops; // every loop around the accumulation, outermost first
    E term;                 // what is added
    std::vector<E> out_index;
    E post;                 // the stored value when it is not the sum itself ((acc / n))
    std::string acc;        // the scalar that accumulates, or "" when the output does
};

void find_sum(Ctx &c, const std::vector<Stmt> &body, std::vector<std::pair<std::string, int64_t>> &stack, std::vector<SumNest> &found, std::map<std::string, E> &env)
{
    const int out = (int)c.k.inputs.size();
    for (auto &s : body) {
        if (s.kind == Stmt::For) {
            stack.push_back({s.var, s.bound});
            find_sum(c, s.body, stack, found, env);
            stack.pop_back();
        } else if (s.kind == Stmt::Set && s.var[0] == 's') {
            const E &v = s.value;
            if (is_bin(v, "+") && v->kids[0]->kind == Expr::Var && v->kids[0]->text == s.var) {
                SumNest n;
                n.loops = stack;
                n.term = v->kids[1];
                n.acc = s.var;
                found.push_back(n);
            } else if (v->kind == Expr::Load && !v->vec) {
                env[s.var] = v; // s0 = %0[i0, i1]: a loaded value kept for the loop below it
            }
        } else if (s.kind == Stmt::Store && s.buf == out && !s.vec) {
            const E &v = s.value;
            bool into_itself = is_bin(v, "+") && v->kids[0]->kind == Expr::Load && v->kids[0]->buf == out && v->kids[0]->kids.size() == s.index.size();
            for (size_t i = 0; into_itself && i < s.index.size(); ++i) into_itself = same(v->kids[0]->kids[i], s.index[i]);
            if (into_itself) {
                SumNest n;
                n.loops = stack;
                n.term = v->kids[1];
                n.out_index = s.index;
                found.push_back(n);
            } else if (!found.empty() && !found.back().acc.empty() && found.back().out_index.empty()) {
                // the store of a scalar's sum: the sum itself or (acc / n)
                SumNest &n = found.back();
                bool plain = v->kind == Expr::Var && v->text == n.acc;
                bool mean = is_bin(v, "/") && v->kids[0]->kind == Expr::Var && v->kids[0]->text == n.acc && v->kids[1]->kind == Expr::Num;
                if (plain || mean) {
                    n.out_index = s.index;
                    if (mean) n.post = v;
                }
            }
        }
    }
}

bool try_sum(Ctx &c)
{
    std::vector<SumNest> found;
    std::vector<std::pair<std::string, int64_t>> stack;
    std::map<std::string, E> env;
    find_sum(c, c.k.body, stack, found, env);
    if (found.size() != 1) return false;
    SumNest &n = found[0];
    if (n.out_index.size() != c.k.output.dims.size()) return false;
    const int out = (int)c.k.inputs.size();
    // the output's axes: the loops its store is indexed by, in the output's order; the rest are summed, in nesting order
    set_dims_from_output(c);
    std::set<std::string> outer;
    for (size_t a = 0; a < n.out_index.size(); ++a) {
        const E &ix = n.out_index[a];
        if (ix->kind != Expr::Var || ix->text[0] != 'i') refuse(PSK_E7005, c.k.name + ": the sum's store is indexed by `" + show(ix) + "`, not by a loop");
        c.pos[ix->text] = (int)a;
        outer.insert(ix->text);
    }
    int inner = 0;
    for (auto &lp : n.loops) {
        if (outer.count(lp.first)) {
            if (lp.second != c.k.output.dims[c.pos[lp.first]]) refuse(PSK_E7001, c.k.name + ": the loop " + lp.first + " does not run over its output axis");
            continue;
        }
        if (inner >= PSK_MAX_INNER) refuse(PSK_E7005, c.k.name + ": more summed axes than a launch holds");
        c.pos[lp.first] = c.l.n_outer + inner;
        c.l.dims[c.l.n_outer + inner] = lp.second;
        ++inner;
    }
    for (auto &v : outer) {
        bool looped = false;
        for (auto &lp : n.loops) looped |= lp.first == v;
        if (!looped) refuse(PSK_E7005, c.k.name + ": the output index " + v + " is no loop around the sum");
    }
    c.l.n_inner = inner;
    c.naxes = c.l.n_outer + inner;
    c.scalars = env;
    c.set_operand(c.l.out, out, n.out_index);
    // the term: a load (a reduction), a load squared (sum_squares), or a product of two loads (a contraction),
    // the generic `ein`'s leading (1 * x0) included
    auto resolve = [&](E e) -> E {
        if (e->kind == Expr::Var && e->text[0] == 's') {
            auto it = env.find(e->text);
            if (it != env.end()) return it->second;
        }
        if (is_bin(e, "*") && is_num(e->kids[0], 1.0)) return e->kids[1]; // exact: 1·x
        return e;
    };
    E t = resolve(n.term);
    if (t->kind == Expr::Load && !t->vec) {
        c.use_input(t->buf, t->kids);
        c.l.op = PSK_OP_REDUCE;
        c.l.kind = n.post ? PSK_REDUCE_MEAN : PSK_REDUCE_SUM;
        int64_t count = 1;
        for (int a = 0; a < inner; ++a) count *= c.l.dims[c.l.n_outer + a];
        c.l.iparam[0] = count;
        if (n.post && n.post->kids[1]->num != (double)count) refuse(PSK_E7005, c.k.name + ": a sum divided by something other than its number of terms");
        if (c.k.inputs.size() != 1) refuse(PSK_E7005, c.k.name + ": a reduction of more than one input");
        return true;
    }
    if (is_bin(t, "*")) {
        E a = resolve(t->kids[0]), b = resolve(t->kids[1]);
        if (n.post) refuse(PSK_E7005, c.k.name + ": a contraction whose sum is divided before it is stored");
        if (a->kind == Expr::Load && b->kind == Expr::Load && !a->vec && !b->vec) {
            if (c.k.inputs.size() == 1 && a->buf == 0 && b->buf == 0 && same(a, b)) {
                c.use_input(0, a->kids);
                c.l.op = PSK_OP_REDUCE;
                c.l.kind = PSK_REDUCE_SUMSQ;
                int64_t count = 1;
                for (int x = 0; x < inner; ++x) count *= c.l.dims[c.l.n_outer + x];
                c.l.iparam[0] = count;
                return true;
            }
            if (c.k.inputs.size() != 2 || a->buf != 0 || b->buf != 1) refuse(PSK_E7005, c.k.name + ": a contraction is the product of input 0 and input 1; this one multiplies " + show(a) + " and " + show(b));
            c.use_input(0, a->kids);
            c.use_input(1, b->kids);
            c.l.op = PSK_OP_CONTRACT;
            return true;
        }
        refuse(PSK_E7005, c.k.name + ": a sum of products of more than two operands (or of something other than loads): " + show(t));
    }
    refuse(PSK_E7005, c.k.name + ": a sum of terms this executor has no launch for: " + show(t));
}

// -- by name: functions whose every layout is the same function ----------------------------------------------------
int axis_named(const Buf &b, const std::string &name)
{
    for (size_t i = 0; i < b.names.size(); ++i)
        if (b.names[i] == name) return (int)i;
    return -1;
}

// The first load of buffer `b` anywhere in the nest.
E first_load(const std::vector<Stmt> &body, int b)
{
    E hit;
    auto scan = [&](const E &e, auto &&self) -> void {
        if (!e || hit) return;
        if (e->kind == Expr::Load && e->buf == b) { hit = e; return; }
        for (auto &k : e->kids) self(k, self);
    };
    for (auto &s : body) {
        scan(s.value, scan);
        for (auto &i : s.index) scan(i, scan);
        if (!hit) hit = first_load(s.body, b);
        if (hit) break;
    }
    return hit;
}

void whole(Ctx &c, psk_operand &o, int b, const std::vector<int> &map)
{
    // buffer b row-major, its axis i at position map[i] of the space
    const Buf &s = c.buf(b);
    memset(&o, 0, sizeof o);
    o.dtype = dtype_of(s.type);
    if (o.dtype < 0) refuse(PSK_E7005, c.k.name + ": a buffer of type `" + s.type + "` is not one this executor stores");
    o.is_index = o.dtype == PSK_I64 ? 1 : 0;
    o.numel = s.numel();
    auto st = s.strides();
    for (size_t i = 0; i < map.size(); ++i) o.stride[map[i]] += st[i];
}

bool try_named(Ctx &c)
{
    const Kernel &k = c.k;
    const int out = (int)k.inputs.size();
    if (k.name == "dot" && k.inputs.size() == 2) {
        // x[.., K] · w[K, rest..] (lower.rs:481-513) in any tiling: outer = x's leading axes then w's trailing ones
        const Buf &x = k.inputs[0], &w = k.inputs[1];
        if (x.dims.empty() || w.dims.empty() || x.dims.back() != w.dims[0]) refuse(PSK_E7001, "dot: the contracted axes differ");
        if (k.output.dims.size() != x.dims.size() - 1 + w.dims.size() - 1) refuse(PSK_E7001, "dot: the result's rank is not its operands'");
        set_dims_from_output(c);
        c.l.n_inner = 1;
        c.l.dims[c.l.n_outer] = x.dims.back();
        std::vector<int> mx, mw, mo;
        for (size_t i = 0; i + 1 < x.dims.size(); ++i) mx.push_back((int)i);
        mx.push_back(c.l.n_outer);
        mw.push_back(c.l.n_outer);
        for (size_t i = 1; i < w.dims.size(); ++i) mw.push_back((int)(x.dims.size() - 1 + i - 1));
        for (int i = 0; i < c.l.n_outer; ++i) mo.push_back(i);
        whole(c, c.l.in[0], 0, mx);
        whole(c, c.l.in[1], 1, mw);
        whole(c, c.l.out, out, mo);
        if (w.quant_over >= 0) {
            // the scales: one per index of w's axes outside [over, end), row-major over them
            int64_t acc = 1;
            for (int a = (int)w.dims.size() - 1; a >= 0; --a)
                if (a < w.quant_over || a >= w.quant_end) { c.l.in[1].scale_stride[mw[a]] += acc; acc *= w.dims[a]; }
        }
        c.l.op = PSK_OP_CONTRACT;
        return true;
    }
    if (k.name.compare(0, 13, "softmax axis ") == 0) {
        std::string axis = k.name.substr(13);
        bool masked = false;
        size_t wh = axis.find(" where");
        if (wh != std::string::npos) { masked = true; if (axis.substr(wh) != " where") refuse(PSK_E7005, k.name + ": only the three-pass forms are known"); axis = axis.substr(0, wh); }
        if (k.inputs.size() != (masked ? 2u : 1u)) refuse(PSK_E7001, k.name + ": one input, and a mask after `where`");
        const Buf &x = k.inputs[0];
        const int p = axis_named(x, axis);
        if (p < 0 || x.dims != k.output.dims) refuse(PSK_E7001, k.name + ": no axis `" + axis + "` in the input, or a result of another shape");
        if (x.dims.size() - 1 > PSK_MAX_RANK) refuse(PSK_E7005, k.name + ": more axes than a launch holds");
        c.l.n_outer = (int)x.dims.size() - 1;
        c.l.n_inner = 1;
        std::vector<int> map;
        for (int i = 0, o = 0; i < (int)x.dims.size(); ++i) {
            if (i == p) { map.push_back(c.l.n_outer); c.l.dims[c.l.n_outer] = x.dims[i]; }
            else { c.l.dims[o] = x.dims[i]; map.push_back(o++); }
        }
        whole(c, c.l.in[0], 0, map);
        whole(c, c.l.out, out, map);
        if (masked) {
            // the mask's axes are those of the input it is read by in the nest: %1[i.., ..] names the input's loops
            E ld = first_load(k.body, 1), lx = first_load(k.body, 0);
            if (!ld || !lx || lx->kids.size() != x.dims.size()) refuse(PSK_E7005, k.name + ": the nest reads no mask");
            std::vector<int> mm;
            for (auto &ix : ld->kids) {
                int at = -1;
                for (size_t i = 0; i < lx->kids.size(); ++i)
                    if (same(lx->kids[i], ix)) at = (int)i;
                if (at < 0) refuse(PSK_E7005, k.name + ": the mask is indexed by `" + show(ix) + "`, which does not index the input");
                mm.push_back(map[at]);
            }
            whole(c, c.l.in[1], 1, mm);
            c.l.masked = 1;
        }
        c.l.op = PSK_OP_SOFTMAX;
        return true;
    }
    if (k.name == "cross_entropy" && k.inputs.size() == 2) {
        const Buf &lg = k.inputs[0], &y = k.inputs[1];
        if (lg.dims.size() != y.dims.size() + 1 || k.output.dims != y.dims) refuse(PSK_E7001, "cross_entropy: logits [.., classes] against labels [..]");
        set_dims_from_output(c);
        c.l.n_inner = 1;
        c.l.dims[c.l.n_outer] = lg.dims.back();
        std::vector<int> ml, my;
        for (int i = 0; i < (int)lg.dims.size(); ++i) ml.push_back(i);
        for (int i = 0; i < (int)y.dims.size(); ++i) my.push_back(i);
        whole(c, c.l.in[0], 0, ml);
        whole(c, c.l.in[1], 1, my);
        whole(c, c.l.out, out, my);
        c.l.op = PSK_OP_XENT;
        return true;
    }
    if (k.name == "argmax" && k.inputs.size() == 1) {
        const Buf &x = k.inputs[0];
        if (x.dims.empty() || x.dims.size() != k.output.dims.size() + 1) refuse(PSK_E7001, "argmax: the last axis of the input is the one searched");
        set_dims_from_output(c);
        c.l.n_inner = 1;
        c.l.dims[c.l.n_outer] = x.dims.back();
        std::vector<int> mx, mo;
        for (int i = 0; i < (int)x.dims.size(); ++i) mx.push_back(i);
        for (int i = 0; i + 1 < (int)x.dims.size(); ++i) mo.push_back(i);
        whole(c, c.l.in[0], 0, mx);
        whole(c, c.l.out, out, mo);
        c.l.op = PSK_OP_ARGMAX;
        return true;
    }
    if (k.name == "embed" && k.inputs.size() == 2) {
        // out[ix.., j] = table[idx[ix..], j] (lower.rs:1421-1437)
        const Buf &t = k.inputs[0], &ix = k.inputs[1];
        if (t.dims.size() != 2 || k.output.dims.size() != ix.dims.size() + 1 || k.output.dims.back() != t.dims[1]) refuse(PSK_E7001, "embed: a table [rows, d] and indices; the result is the indices' shape and d");
        set_dims_from_output(c);
        std::vector<int> mi, mo;
        for (int i = 0; i < (int)ix.dims.size(); ++i) mi.push_back(i);
        for (int i = 0; i < (int)k.output.dims.size(); ++i) mo.push_back(i);
        whole(c, c.l.in[1], 1, mi);
        whole(c, c.l.out, out, mo);
        // the table: its row is chosen by the index, its columns walk the last axis
        memset(&c.l.in[0], 0, sizeof c.l.in[0]);
        c.l.in[0].dtype = dtype_of(t.type);
        if (c.l.in[0].dtype < 0) refuse(PSK_E7005, "embed: a table of type `" + t.type + "`");
        c.l.in[0].numel = t.numel();
        c.l.in[0].stride[0] = t.dims[1]; // a row of the table, then its columns: the table is indexed by the
        c.l.in[0].stride[1] = 1;         // loaded index, not by the space, so these two words are its two strides
        c.l.iparam[0] = t.dims[0];
        c.l.op = PSK_OP_EMBED;
        return true;
    }
    return false;
}

void describe(const Kernel &k, int order, psk_launch &l)
{
    memset(&l, 0, sizeof l);
    if (k.formats) refuse(PSK_E7005, k.name + ": the kernel states arithmetic formats of its own; those are the kernel interpreter's to emulate, this executor computes in f32");
    const int d = dtype_of(k.output.type);
    if (d < 0) refuse(PSK_E7005, k.name + ": a result of type `" + k.output.type + "` is not one this executor stores");
    if (k.inputs.size() > PSK_MAX_INPUTS) refuse(PSK_E7005, k.name + ": more inputs than a launch holds");
    // the kernel's own type: that of its real buffers (an index result comes from a kernel over reals or indices)
    int kd = d;
    if (d == PSK_I64)
        for (auto &b : k.inputs) { int t = dtype_of(b.type); if (t >= 0 && t != PSK_I64 && t != PSK_I8) { kd = t; break; } }
    l.dtype = kd == PSK_I64 ? PSK_F32 : kd;
    l.order = order;
    l.guarded = 1;
    l.n_inputs = (int)k.inputs.size();
    const bool vec = has_vector(k.body);
    // nests with a loaded index or a data-dependent scan are known by their names; the rest by their structure
    const bool by_name = k.name.compare(0, 13, "softmax axis ") == 0 || k.name == "cross_entropy" || k.name == "argmax" || k.name == "embed";
    auto fresh = [&]() {
        const int kd2 = l.dtype;
        memset(&l, 0, sizeof l);
        l.dtype = kd2; l.order = order; l.guarded = 1; l.n_inputs = (int)k.inputs.size();
    };
    bool ok = false;
    if (!vec && !by_name) {
        Ctx c(k, l);
        ok = try_elementwise(c);
        if (!ok) {
            fresh();
            Ctx c2(k, l);
            ok = try_sum(c2);
        }
        if (!ok) fresh();
    }
    if (!ok) {
        Ctx c3(k, l);
        ok = try_named(c3);
    }
    if (!ok) refuse(PSK_E7005, k.name + ": this executor has no launch for this nest" + (vec ? " (a tiled or laned form of something other than `dot`)" : ""));
    if (l.out.dtype == PSK_I64) l.out.is_index = 1;
}

} // namespace

extern "C" int psk_describe(const char *kernel_text, int32_t order, psk_launch *out, char *name, size_t name_cap, const char **rest, char *err, size_t err_cap)
{
    if (err && err_cap) err[0] = 0;
    if (!kernel_text || !out) {
        if (err && err_cap) snprintf(err, err_cap, "psk_describe: a null argument");
        return PSK_E7001;
    }
    try {
        Kernel k = read_kernel(kernel_text, rest);
        describe(k, order == PSK_ORDER_DEVICE ? PSK_ORDER_DEVICE : PSK_ORDER_SEQUENTIAL, *out);
        if (name && name_cap) {
            snprintf(name, name_cap, "%s", k.name.c_str());
            out->name = name;
        } else {
            out->name = nullptr;
        }
        return PSK_OK;
    } catch (const Refuse &r) {
        if (err && err_cap) snprintf(err, err_cap, "%s", r.msg.c_str());
        return r.code;
    } catch (const std::exception &e) {
        if (err && err_cap) snprintf(err, err_cap, "psk_describe: %s", e.what());
        return PSK_E10001;
    }
}
