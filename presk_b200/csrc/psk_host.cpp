// The host program: what the reference's `KernelBackend` does between
// `Backend::call` and the executor (crates/presk-kernel/src/host.rs:436-457,
// 742-868, 887-1039). It walks a model's lets in the reference's order, forms
// the fusion groups of presk-core/src/fusion.rs:138-, looks each site's
// storage type up in the realization (presk-rt/src/lib.rs:459-471), allocates
// the output, and hands the executor one launch per group or tensor primitive.
// It runs over any executor given as a table of functions, as
// `KernelBackend::with_exec` does (host.rs:466).
//
// The reference walks PSK-Core, which its front end produces from a `.psk`
// source; that front end is not part of this library, so the models this file
// knows are written out here let by let, each function numbering its
// parameters and then every let as presk-core's lowering does
// (crates/presk-core/tests/snapshots/lower__core_minigpt.snap shows the rule),
// so that a site is "<function>/%<let>" as in the reference's realization
// files.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/presk_cuda.h"

namespace {

std::string g_host_error;

struct HostError {
    int code;
    std::string msg;
};

[[noreturn]] void raise(int code, const std::string &m) { throw HostError{code, m}; }

size_t elem_bytes(int dtype)
{
    switch (dtype) {
    case PSK_F64: case PSK_I64: return 8;
    case PSK_F32: return 4;
    case PSK_BF16: case PSK_F16: return 2;
    case PSK_E8M15: return 3;
    default: return 1;
    }
}

int dtype_of_name(const std::string &s)
{
    if (s == "f64") return PSK_F64;
    if (s == "f32") return PSK_F32;
    if (s == "bf16") return PSK_BF16;
    if (s == "f16") return PSK_F16;
    if (s == "e8m15") return PSK_E8M15;
    if (s == "e4m3fn" || s == "e4m3") return PSK_E4M3;
    return -1;
}

// ---- a reader of the realization's JSON: objects, strings, numbers ----------
struct Json {
    enum Kind { Null, Str, Num, Obj } kind = Null;
    std::string str;
    double num = 0;
    std::vector<std::pair<std::string, Json>> obj;
    const Json *get(const std::string &k) const
    {
        for (auto &kv : obj)
            if (kv.first == k) return &kv.second;
        return nullptr;
    }
};

struct JsonReader {
    const char *p;
    explicit JsonReader(const char *s) : p(s) {}
    void ws() { while (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r') ++p; }
    std::string string()
    {
        std::string s;
        ++p;
        while (*p && *p != '"') {
            if (*p == '\\' && p[1] == 'u' && p[2] && p[3] && p[4] && p[5]) {
                // a \uXXXX escape of the basic plane, as UTF-8 (parameter paths hold γ and β)
                unsigned cp = (unsigned)strtoul(std::string(p + 2, 4).c_str(), nullptr, 16);
                if (cp < 0x80) s.push_back((char)cp);
                else if (cp < 0x800) { s.push_back((char)(0xc0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3f))); }
                else { s.push_back((char)(0xe0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3f))); s.push_back((char)(0x80 | (cp & 0x3f))); }
                p += 6;
                continue;
            }
            if (*p == '\\' && p[1]) ++p;
            s.push_back(*p++);
        }
        if (*p != '"') raise(PSK_E7001, "realization: an unterminated string");
        ++p;
        return s;
    }
    Json value()
    {
        ws();
        Json j;
        if (*p == '{') {
            j.kind = Json::Obj;
            ++p;
            ws();
            if (*p == '}') { ++p; return j; }
            for (;;) {
                ws();
                if (*p != '"') raise(PSK_E7001, "realization: a key was expected");
                std::string k = string();
                ws();
                if (*p != ':') raise(PSK_E7001, "realization: `:` was expected after a key");
                ++p;
                j.obj.emplace_back(k, value());
                ws();
                if (*p == ',') { ++p; continue; }
                if (*p == '}') { ++p; break; }
                raise(PSK_E7001, "realization: `,` or `}` was expected");
            }
        } else if (*p == '"') {
            j.kind = Json::Str;
            j.str = string();
        } else if (*p == '-' || (*p >= '0' && *p <= '9')) {
            char *end;
            j.kind = Json::Num;
            j.num = strtod(p, &end);
            p = end;
        } else if (!strncmp(p, "null", 4)) {
            p += 4;
        } else if (!strncmp(p, "true", 4)) {
            p += 4; j.kind = Json::Num; j.num = 1;
        } else if (!strncmp(p, "false", 5)) {
            p += 5; j.kind = Json::Num; j.num = 0;
        } else {
            raise(PSK_E7001, "realization: not JSON this reader takes");
        }
        return j;
    }
};

struct QuantSpec {
    int bits = 8;
    int over = 0;
};

// presk-rt/src/lib.rs:374-434, the fields this executor reads.
struct Realization {
    int dflt = PSK_F32;
    std::map<std::string, int> storage, functions, params;
    std::map<std::string, QuantSpec> quant;
    struct AffineSpec { int kind; float scale; int zero; };
    std::map<std::string, AffineSpec> scaled;  // sites stored in an affine format (presk-rt/src/lib.rs:287-360)
    std::map<std::string, int> int_sums;        // sites whose `product` and `accum` are i32: 1 product, 2 accum, 3 both
    int order = PSK_ORDER_SEQUENTIAL;
    int order_size = 0;               // chunked(size)
    bool blockwise_attention = false; // "order": {"kind": "device", "attention": "blockwise"} or "online"
    bool online_attention = false;    // "attention": "online": the one-pass form of the same launch
    bool merged_launches = false;     // "order": {..., "launches": "merged"}: bit-preserving rewrites of the launch list

    static Realization parse(const char *text)
    {
        Realization r;
        std::string t(text ? text : "f32");
        size_t a = t.find_first_not_of(" \n\t\r");
        if (a == std::string::npos) raise(PSK_E7001, "realization: empty");
        if (t[a] != '{') {
            size_t b = t.find_last_not_of(" \n\t\r");
            int d = dtype_of_name(t.substr(a, b - a + 1));
            if (d < 0) raise(PSK_E7001, "realization: no type `" + t + "`");
            r.dflt = d;
            return r;
        }
        JsonReader rd(t.c_str());
        Json j = rd.value();
        auto dt = [](const Json &v, const std::string &what) {
            int d = v.kind == Json::Str ? dtype_of_name(v.str) : -1;
            if (d < 0) raise(PSK_E7001, "realization: " + what + " names no type this executor stores");
            return d;
        };
        if (auto *d = j.get("default")) r.dflt = dt(*d, "default");
        for (auto key : {"storage", "functions", "params"}) {
            if (auto *m = j.get(key)) {
                auto &dst = std::string(key) == "storage" ? r.storage : std::string(key) == "functions" ? r.functions : r.params;
                for (auto &kv : m->obj) dst[kv.first] = dt(kv.second, std::string(key) + "[" + kv.first + "]");
            }
        }
        if (auto *q = j.get("quant"))
            for (auto &kv : q->obj) {
                QuantSpec s;
                if (auto *b = kv.second.get("bits")) s.bits = (int)b->num;
                // `over` is an AxisRef: a position or a name (presk-rt/src/quant.rs:46-49). Parameters reach this
                // host without axis names (psk_host_set_param takes lengths only), so a name cannot be resolved here.
                const Json *o = kv.second.get("over");
                if (!o) raise(PSK_E7001, "realization: quant[" + kv.first + "] names no axis (`over`)");
                if (o->kind != Json::Num) raise(PSK_E7005, "realization: quant[" + kv.first + "]: `over` is given by position on this executor (its parameters carry no axis names)");
                s.over = (int)o->num;
                if (s.bits != 8) raise(PSK_E7005, "realization: quant[" + kv.first + "]: this executor stores int8 weights only");
                // the scales are absmax ones (quant.rs:299-323 `scale_of`); a power-of-two scheme gives other codes
                if (const Json *sc = kv.second.get("scheme"))
                    if (sc->kind != Json::Str || sc->str != "absmax")
                        raise(PSK_E7005, "realization: quant[" + kv.first + "]: the scheme `" + (sc->kind == Json::Str ? sc->str : "?") + "` is not one this executor quantises with (absmax)");
                r.quant[kv.first] = s;
            }
        if (auto *o = j.get("order")) {
            const Json *k = o->get("kind");
            std::string kind = k ? k->str : "sequential";
            if (kind == "sequential" || kind == "blocked") r.order = PSK_ORDER_SEQUENTIAL;
            else if (kind == "device") r.order = PSK_ORDER_DEVICE;
            else if (kind == "chunked") {
                // presk-rt/src/lib.rs:264-269: sums of `size` consecutive terms, then the chunks' sums
                const Json *sz = o->get("size");
                if (!sz || sz->kind != Json::Num || sz->num < 1 || sz->num != std::floor(sz->num) || sz->num > 2147483647.0) raise(PSK_E7001, "realization: the order chunked needs a whole `size` of at least 1");
                r.order = PSK_ORDER_CHUNKED;
                r.order_size = (int)sz->num;
            }
            else raise(PSK_E7005, "realization: the order `" + kind + "` is not one this executor has kernels for (sequential, chunked, device)");
            if (const Json *ml = o->get("launches")) {
                if (ml->str == "merged") r.merged_launches = true;
                else if (ml->str != "reference") raise(PSK_E7005, "realization: the launch list `" + ml->str + "` is not one this executor has (reference, merged)");
            }
            if (const Json *at = o->get("attention")) {
                if (at->str == "blockwise") {
                    if (r.order != PSK_ORDER_DEVICE) raise(PSK_E7005, "realization: `attention: blockwise` is part of the order `device`");
                    r.blockwise_attention = true;
                } else if (at->str == "online") {
                    if (r.order != PSK_ORDER_DEVICE) raise(PSK_E7005, "realization: `attention: online` is part of the order `device`");
                    r.blockwise_attention = true;
                    r.online_attention = true;
                } else if (at->str != "unfused") {
                    raise(PSK_E7005, "realization: the attention order `" + at->str + "` is not one this executor has (unfused, blockwise, online)");
                }
            }
        }
        if (auto *m = j.get("arith"))
            if (!m->obj.empty()) raise(PSK_E7005, "realization: `arith` formats are the kernel interpreter's; this executor computes in f32 (E7005)");
        for (auto key : {"product", "accum"})
            if (auto *m = j.get(key))
                for (auto &kv : m->obj) {
                    if (kv.second.kind != Json::Str || kv.second.str != "i32")
                        raise(PSK_E7005, std::string("realization: ") + key + "[" + kv.first + "]: this executor counts sums in i32 (wrapping) only (E7005)");
                    r.int_sums[kv.first] |= std::string(key) == "product" ? 1 : 2;
                }
        for (auto &kv : r.int_sums)
            if (kv.second != 3) raise(PSK_E7005, "realization: " + kv.first + ": `product` and `accum` are i32 together on this executor (E7005)");
        if (auto *m = j.get("scaled"))
            for (auto &kv : m->obj) {
                const Json *i = kv.second.get("int"), *sc = kv.second.get("scale"), *z = kv.second.get("zero");
                // a scheme whose scale is not computed yet is refused by every executor (E7006, presk-rt/src/lib.rs:544-549)
                if (!sc || sc->kind != Json::Num) raise(PSK_E7006, "realization: scaled[" + kv.first + "] has no scale yet: `presk scales` computes it from an envelope (E7006)");
                AffineSpec a;
                std::string in = i && i->kind == Json::Str ? i->str : "";
                if (in == "i8/sat") a.kind = 1;
                else if (in == "u8/sat") a.kind = 2;
                else raise(PSK_E7005, "realization: scaled[" + kv.first + "]: the codes are i8/sat or u8/sat on this executor (E7005)");
                a.scale = (float)sc->num;
                a.zero = z ? (int)z->num : 0;
                if (!(a.scale > 0.0f) || !std::isnormal(a.scale)) raise(PSK_E7001, "realization: scaled[" + kv.first + "]: the scale is a positive normal binary32 number");
                if (a.zero < (a.kind == 2 ? 0 : -128) || a.zero > (a.kind == 2 ? 255 : 127)) raise(PSK_E7001, "realization: scaled[" + kv.first + "]: the zero point is not one of its codes");
                r.scaled[kv.first] = a;
            }
        return r;
    }

    // Realization::dtype_at: the site's own type, else its function's, else the default.
    int dtype_at(const std::string &site) const
    {
        auto it = storage.find(site);
        if (it != storage.end()) return it->second;
        size_t slash = site.rfind('/');
        if (slash != std::string::npos) {
            auto f = functions.find(site.substr(0, slash));
            if (f != functions.end()) return f->second;
        }
        return dflt;
    }
};

// ---- values -------------------------------------------------------------------
struct Storage {
    const psk_exec_vtable *vt;
    void *p;
    size_t bytes;
    Storage(const psk_exec_vtable *v, size_t b) : vt(v), p(v->alloc(v->self, b)), bytes(b)
    {
        if (!p) raise(PSK_E10001, std::string("the executor could not allocate ") + std::to_string(b) + " bytes: " + v->last_error(v->self));
    }
    ~Storage() { vt->free(vt->self, p); }
    Storage(const Storage &) = delete;
};

struct Axis {
    std::string name; // empty: unnamed
    int64_t len;
};

typedef std::vector<Axis> Axes;

// A tensor on the executor: row-major over its axes from an element offset.
struct Tensor {
    std::shared_ptr<Storage> st;
    int64_t off = 0;
    Axes axes;
    int dtype = PSK_F32;
    bool is_index = false;
    int64_t bound = 0;
    // integer weights: scales over the axes without `q_over`
    std::shared_ptr<Storage> scales;
    int64_t soff = 0;
    int affine = 0;  // the value is stored in an affine format: 1 i8/sat, 2 u8/sat
    int affine_zero = 0;
    float affine_scale = 0.0f;
    int q_over = -1; // the first axis of the contracted one, and how many axes it has been split into
    int q_span = 1;
    bool borrowed = false;
    void *raw = nullptr; // a caller's device buffer (psk_host_call_device)
    std::vector<int64_t> vstrides; // a view that is not row-major over its axes (merged launches only); empty: row-major

    int64_t numel() const { int64_t n = 1; for (auto &a : axes) n *= a.len; return n; }
    void *ptr() const { return raw ? raw : st->p; }
    std::vector<int64_t> strides() const
    {
        if (!vstrides.empty()) return vstrides;
        std::vector<int64_t> s(axes.size());
        int64_t acc = 1;
        for (int i = (int)axes.size() - 1; i >= 0; --i) { s[i] = acc; acc *= axes[i].len; }
        return s;
    }
    std::vector<int64_t> scale_strides() const
    {
        std::vector<int64_t> s(axes.size(), 0);
        if (q_over < 0) return s;
        int64_t acc = 1;
        for (int i = (int)axes.size() - 1; i >= 0; --i) {
            if (i >= q_over && i < q_over + q_span) continue;
            s[i] = acc;
            acc *= axes[i].len;
        }
        return s;
    }
};

std::string show(const Axes &a)
{
    std::string s = "[";
    for (size_t i = 0; i < a.size(); ++i) {
        if (i) s += ", ";
        s += a[i].name.empty() ? std::to_string(a[i].len) : a[i].name + ": " + std::to_string(a[i].len);
    }
    return s + "]";
}

// lower.rs:37-56: trailing positions when the names agree, else by name.
bool align(const Axes &src, const Axes &target, std::vector<int> &map)
{
    map.clear();
    if (src.size() > target.size()) return false;
    size_t off = target.size() - src.size();
    bool positional = true;
    for (size_t i = 0; i < src.size() && positional; ++i) {
        const Axis &t = target[off + i];
        positional = src[i].len == t.len && (src[i].name.empty() || t.name.empty() || src[i].name == t.name);
    }
    if (positional) {
        for (size_t i = 0; i < src.size(); ++i) map.push_back((int)(off + i));
        return true;
    }
    for (auto &a : src) {
        if (a.name.empty()) return false;
        int p = -1;
        for (size_t k = 0; k < target.size(); ++k)
            if (target[k].name == a.name && target[k].len == a.len) { p = (int)k; break; }
        if (p < 0) return false;
        map.push_back(p);
    }
    return true;
}

// lower.rs:59-70
bool result_axes(const Axes &a, const Axes &b, Axes &out)
{
    const Axes &lng = a.size() >= b.size() ? a : b, &sht = a.size() >= b.size() ? b : a;
    std::vector<int> map;
    if (!align(sht, lng, map)) return false;
    out = lng;
    for (size_t i = 0; i < map.size(); ++i)
        if (out[map[i]].name.empty()) out[map[i]].name = sht[i].name;
    return true;
}

const char *prim_name(int p)
{
    static const char *n[] = {"add", "sub", "mul", "div", "max", "min", "neg", "exp", "log", "tanh", "sqrt", "sin", "cos", "abs", "gelu", "gelu_deriv", "relu", "heaviside", "sign", "sigmoid", "pow", "real", "div_n", "round"};
    return n[p];
}

struct StepSpec {
    int prim;
    int a, b; // sources: >= 0 an input of the group, < 0 step -1-k; b unused when unary
    int imm;
    bool unary;
};

StepSpec U(int prim, int a, int imm = 0) { return {prim, a, 0, imm, true}; }
StepSpec Bn(int prim, int a, int b) { return {prim, a, b, 0, false}; }
inline int S(int k) { return -1 - k; } // the value of step k

} // namespace

// ===========================================================================
struct psk_host {
    const psk_exec_vtable *vt;
    psk_exec_vtable vt_copy;
    Realization rz;
    std::string error;
    std::string model;
    std::map<std::string, int64_t> consts;
    std::map<std::string, Tensor> params;
    int64_t launches = 0;
    // calibration: one slot of four words a site, on the executor (PSK_OP_MAGNITUDE)
    bool calibrating = false;
    std::map<std::string, int> slot_of;
    std::shared_ptr<Storage> slots;
    static constexpr int kMaxSites = 4096;
    std::string current_site;
    std::string envelope_text;
    bool logging = false;
    std::string log;
    Tensor last_result;

    int64_t C(const std::string &k) const
    {
        auto it = consts.find(k);
        if (it == consts.end()) raise(PSK_E7001, "the constant `" + k + "` was not given");
        return it->second;
    }
    int64_t C(const std::string &k, int64_t dflt) const
    {
        auto it = consts.find(k);
        return it == consts.end() ? dflt : it->second;
    }

    // ---- buffers --------------------------------------------------------------
    Tensor fresh(const Axes &axes, int dtype, bool is_index = false, int64_t bound = 0)
    {
        Tensor t;
        t.axes = axes;
        t.dtype = is_index ? PSK_I64 : dtype;
        t.is_index = is_index;
        t.bound = bound;
        t.st = std::make_shared<Storage>(vt, (size_t)std::max<int64_t>(1, t.numel()) * elem_bytes(t.dtype));
        return t;
    }

    // The buffer of a site's value: in its storage type, or in its affine format's codes.
    Tensor fresh_at(const std::string &site, const Axes &axes)
    {
        int d = site_dtype(site);
        auto a = rz.scaled.find(site);
        if (a == rz.scaled.end()) return fresh(axes, d);
        Tensor t = fresh(axes, a->second.kind == 2 ? PSK_U8 : PSK_I8);
        t.affine = a->second.kind;
        t.affine_zero = a->second.zero;
        t.affine_scale = a->second.scale;
        return t;
    }

    void check(int rc, const char *what)
    {
        if (rc != PSK_OK) raise(rc, std::string(what) + ": " + vt->last_error(vt->self));
    }

    // ---- one launch -------------------------------------------------------------
    void set_operand(psk_operand &o, const Tensor &t, const std::vector<int64_t> &stride, const std::vector<int64_t> &sstride)
    {
        memset(&o, 0, sizeof o);
        o.dtype = t.dtype;
        o.is_index = t.is_index ? 1 : 0;
        o.offset = t.off;
        o.numel = t.numel();
        o.affine = t.affine;
        o.affine_zero = t.affine_zero;
        o.affine_scale = t.affine_scale;
        for (size_t a = 0; a < stride.size(); ++a) o.stride[a] = stride[a];
        for (size_t a = 0; a < sstride.size(); ++a) o.scale_stride[a] = sstride[a];
    }

    // `may_refuse`: a merged launch the executor may decline (E7005) before doing anything; the caller
    // then issues the launches it stands for. Returns whether it ran.
    bool run(psk_launch &l, const std::string &name, const std::vector<const Tensor *> &ins, const Tensor &out, bool may_refuse = false)
    {
        l.name = name.c_str();
        l.order = rz.order;
        l.order_size = rz.order_size;
        if (rz.order == PSK_ORDER_CHUNKED && !((l.op == PSK_OP_CONTRACT && l.n_inner == 1 && ins.size() == 2 && !l.int_accum))) {
            // only a contraction of two operands over one summed axis takes a chunked order; every other
            // launch keeps the sequential one (lower.rs:262-266 `chunked(order)`, 429-431)
            if (l.op == PSK_OP_CONTRACT && !l.int_accum && l.n_inner > 1) raise(PSK_E7005, name + ": the order chunked(" + std::to_string(rz.order_size) + ") sums one summed axis in chunks, and this sum runs over " + std::to_string(l.n_inner) + " axes");
            l.order = PSK_ORDER_SEQUENTIAL;
            l.order_size = 0;
        }
        l.guarded = 1;
        l.n_inputs = (int)ins.size();
        std::vector<void *> table;
        for (auto *t : ins) table.push_back(t->ptr());
        table.push_back(out.ptr());
        for (auto *t : ins)
            if (t->dtype == PSK_I8 && !t->affine) table.push_back((uint8_t *)t->scales->p + t->soff * 4);
        int rc = vt->run(vt->self, &l, table.data());
        if (rc == PSK_E7005 && may_refuse) return false;
        check(rc, name.c_str());
        launches += 1;
        if (logging) { log += name; log += '\n'; }
        if (calibrating && !out.is_index && out.numel() > 0 && !current_site.empty()) observe(out);
        return true;
    }

    // Folds a launch's output into its site's magnitudes.
    void observe(const Tensor &out)
    {
        if (!slots) {
            slots = std::make_shared<Storage>(vt, (size_t)kMaxSites * 16);
            std::vector<uint32_t> init((size_t)kMaxSites * 4);
            for (int i = 0; i < kMaxSites; ++i) { init[4 * i] = 0u; init[4 * i + 1] = 0x7f800000u; init[4 * i + 2] = 0xff800000u; init[4 * i + 3] = 0x007fffffu; }
            check(vt->upload(vt->self, slots->p, init.data(), init.size() * 4), "calibrate");
        }
        auto it = slot_of.find(current_site);
        if (it == slot_of.end()) {
            if ((int)slot_of.size() >= kMaxSites) raise(PSK_E7001, "calibrate: more sites than the envelope holds");
            it = slot_of.emplace(current_site, (int)slot_of.size()).first;
        }
        psk_launch m;
        memset(&m, 0, sizeof m);
        m.name = "magnitude";
        m.op = PSK_OP_MAGNITUDE;
        m.dtype = PSK_F32;
        m.n_inputs = 1;
        m.n_outer = 1;
        m.dims[0] = 4;
        set_operand(m.in[0], out, {0}, {0});
        m.out.dtype = PSK_I64; // four raw words; read as integers, never rounded
        m.out.offset = 0;
        m.out.numel = 4;
        m.out.stride[0] = 1;
        void *table[2] = {out.ptr(), (uint8_t *)slots->p + (size_t)it->second * 16};
        check(vt->run(vt->self, &m, table), "magnitude");
    }

    int site_dtype(const std::string &site)
    {
        current_site = site;
        return rz.dtype_at(site);
    }

    // An operand's strides over an iteration space, given where each of its
    // axes sits in it (`map[i]` = position of axis i).
    void view(const Tensor &t, const std::vector<int> &map, int naxes, std::vector<int64_t> &stride, std::vector<int64_t> &sstride)
    {
        stride.assign(naxes, 0);
        sstride.assign(naxes, 0);
        auto st = t.strides(), ss = t.scale_strides();
        for (size_t i = 0; i < map.size(); ++i) {
            stride[map[i]] += st[i];
            sstride[map[i]] += ss[i];
        }
    }

    std::vector<int64_t> contiguous(const Axes &axes)
    {
        Tensor t;
        t.axes = axes;
        return t.strides();
    }

    void set_space(psk_launch &l, const Axes &outer, const std::vector<int64_t> &inner)
    {
        if (outer.size() > PSK_MAX_RANK || inner.size() > PSK_MAX_INNER) raise(PSK_E7001, "a launch of more axes than the executor's descriptor holds");
        l.n_outer = (int)outer.size();
        l.n_inner = (int)inner.size();
        for (size_t a = 0; a < outer.size(); ++a) l.dims[a] = outer[a].len;
        for (size_t c = 0; c < inner.size(); ++c) l.dims[outer.size() + c] = inner[c];
    }

    // ---- host scalars (host.rs:563-591: `self.scalar(x)` = Buf::of(dtype, [x])) --
    std::map<std::pair<std::string, double>, Tensor> scalars;
    Tensor scalar(const std::string &site, double x)
    {
        auto hit = scalars.find({site, x});
        if (hit != scalars.end()) return hit->second;
        int d = site_dtype(site);
        Tensor tmp = fresh({}, PSK_F64);
        check(vt->upload(vt->self, tmp.ptr(), &x, 8), "scalar");
        Tensor out = fresh({}, d);
        convert_into(tmp, out);
        scalars[{site, x}] = out;
        return out;
    }

    void convert_into(const Tensor &src, const Tensor &dst)
    {
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_CONVERT;
        l.dtype = dst.dtype;
        Axes flat = {{"", src.numel()}};
        set_space(l, flat, {});
        set_operand(l.in[0], src, {1}, {0});
        set_operand(l.out, dst, {1}, {0});
        l.order = rz.order == PSK_ORDER_CHUNKED ? PSK_ORDER_SEQUENTIAL : rz.order;
        l.guarded = 1;
        l.n_inputs = 1;
        l.name = "convert";
        void *table[2] = {src.ptr(), dst.ptr()};
        check(vt->run(vt->self, &l, table), "convert");
    }

    // ---- elementwise (lower.rs:309-372) -------------------------------------------
    // `shape`: the result's axes when they are a template's and not the operands' own (mean_vjp broadcasts a
    // cotangent into its template, lower.rs:1257-1270)
    Tensor fused(const std::string &site, const std::vector<StepSpec> &steps, const std::vector<const Tensor *> &ins, const std::string &name_override = "", const Tensor *into = nullptr, const Axes *shape = nullptr)
    {
        // the result's axes: the steps' broadcasts replayed (host.rs:1117-1137)
        std::vector<Axes> shapes;
        for (auto &s : steps) {
            auto of = [&](int src) -> Axes { return src >= 0 ? ins[src]->axes : shapes[-1 - src]; };
            if (s.unary) shapes.push_back(of(s.a));
            else {
                Axes r;
                if (!result_axes(of(s.a), of(s.b), r)) raise(PSK_E7001, std::string("fused: `") + prim_name(s.prim) + "` cannot broadcast " + show(of(s.a)) + " with " + show(of(s.b)));
                shapes.push_back(r);
            }
        }
        Axes out_axes = shape ? *shape : shapes.back();
        int d = site_dtype(site);
        if (into) {
            bool same = into->axes.size() == out_axes.size() && into->dtype == d && !into->affine && !rz.scaled.count(site);
            for (size_t a = 0; same && a < out_axes.size(); ++a) same = into->axes[a].len == out_axes[a].len;
            if (!same) raise(PSK_E7001, "fused: the destination " + show(into->axes) + " is not the group's result " + show(out_axes));
        }
        Tensor out = into ? *into : fresh_at(site, out_axes);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_FUSED;
        l.dtype = d;
        set_space(l, out_axes, {});
        for (size_t i = 0; i < ins.size(); ++i) {
            std::vector<int> map;
            if (!align(ins[i]->axes, out_axes, map)) raise(PSK_E7001, "fused: operand " + std::to_string(i) + " of shape " + show(ins[i]->axes) + " does not broadcast into " + show(out_axes));
            std::vector<int64_t> st, ss;
            view(*ins[i], map, (int)out_axes.size(), st, ss);
            set_operand(l.in[i], *ins[i], st, ss);
        }
        set_operand(l.out, out, out.strides(), {});
        l.n_steps = (int)steps.size();
        for (size_t k = 0; k < steps.size(); ++k) {
            l.steps[k].prim = steps[k].prim;
            l.steps[k].nargs = steps[k].unary ? 1 : 2;
            l.steps[k].src[0] = steps[k].a;
            l.steps[k].src[1] = steps[k].unary ? 0 : steps[k].b;
            l.steps[k].imm = steps[k].imm;
        }
        std::string name = !name_override.empty() ? name_override : steps.size() == 1 ? std::string(prim_name(steps[0].prim)) + (steps[0].prim == PSK_POW ? " " + std::to_string(steps[0].imm) : "") : "fused " + std::to_string(steps.size()) + " steps";
        run(l, name, ins, out);
        return out;
    }

    Tensor unary(const std::string &site, int prim, const Tensor &x, int imm = 0) { return fused(site, {U(prim, 0, imm)}, {&x}); }
    Tensor binary(const std::string &site, int prim, const Tensor &a, const Tensor &b) { return fused(site, {Bn(prim, 0, 1)}, {&a, &b}); }

    // ---- contractions ---------------------------------------------------------------
    // lower.rs:586-636: the iteration space is the output's axes, then the summed
    // ones in the order the operands first name them.
    // `addend`, `add_site`: the residual addition that follows the contraction in the source (`x + f(..)`), issued
    // with it as one launch under merged launches when the executor takes it, else as the `add` it is.
    Tensor ein(const std::string &site, const std::vector<std::string> &output, const std::vector<std::vector<std::string>> &operands, const std::vector<const Tensor *> &ins, const std::string &name_override = "", const Tensor *addend = nullptr, const std::string &add_site = "")
    {
        std::vector<std::pair<std::string, int64_t>> names;
        for (size_t t = 0; t < ins.size(); ++t) {
            if (operands[t].size() != ins[t]->axes.size()) raise(PSK_E7001, "ein: operand " + std::to_string(t) + " has " + std::to_string(ins[t]->axes.size()) + " axes and " + std::to_string(operands[t].size()) + " names");
            for (size_t i = 0; i < operands[t].size(); ++i) {
                bool found = false;
                for (auto &n : names)
                    if (n.first == operands[t][i]) {
                        if (n.second != ins[t]->axes[i].len) raise(PSK_E7001, "ein: axis `" + n.first + "` has lengths " + std::to_string(n.second) + " and " + std::to_string(ins[t]->axes[i].len));
                        found = true;
                    }
                if (!found) names.emplace_back(operands[t][i], ins[t]->axes[i].len);
            }
        }
        Axes out_axes;
        std::vector<std::string> all = output;
        std::vector<int64_t> inner;
        for (auto &o : output) {
            int64_t len = -1;
            for (auto &n : names) if (n.first == o) len = n.second;
            if (len < 0) raise(PSK_E7001, "ein: output axis `" + o + "` appears in no operand");
            out_axes.push_back({o, len});
        }
        for (auto &n : names) {
            bool in_out = false;
            for (auto &o : output) in_out |= o == n.first;
            if (!in_out) { all.push_back(n.first); inner.push_back(n.second); }
        }
        int d = site_dtype(site);
        Tensor out = fresh_at(site, out_axes);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_CONTRACT;
        l.dtype = d;
        l.int_accum = rz.int_sums.count(site) ? 1 : 0;
        set_space(l, out_axes, inner);
        for (size_t t = 0; t < ins.size(); ++t) {
            std::vector<int> map;
            for (auto &n : operands[t])
                for (size_t k = 0; k < all.size(); ++k)
                    if (all[k] == n) { map.push_back((int)k); break; }
            std::vector<int64_t> st, ss;
            view(*ins[t], map, (int)all.size(), st, ss);
            set_operand(l.in[t], *ins[t], st, ss);
        }
        set_operand(l.out, out, contiguous(out_axes), {});
        std::string name = name_override;
        if (name.empty()) {
            name = "ein[";
            for (size_t i = 0; i < output.size(); ++i) name += (i ? ", " : "") + output[i];
            name += "]";
        }
        if (addend && rz.merged_launches && !calibrating && !out.affine && !addend->affine && !rz.scaled.count(add_site)) {
            std::vector<int> amap;
            if (align(addend->axes, out_axes, amap) && addend->axes.size() == out_axes.size()) {
                psk_launch m = l;
                m.op = PSK_OP_CONTRACT_ADD;
                m.iparam[1] = d;
                m.dtype = site_dtype(add_site);
                Tensor sum = fresh(out_axes, m.dtype);
                std::vector<int64_t> st, ss;
                view(*addend, amap, (int)all.size(), st, ss);
                set_operand(m.in[2], *addend, st, ss);
                set_operand(m.out, sum, contiguous(out_axes), {});
                std::vector<const Tensor *> ins3 = ins;
                ins3.push_back(addend);
                if (run(m, name + "+add", ins3, sum, true)) return sum;
                site_dtype(site);
            }
        }
        run(l, name, ins, out);
        if (addend) return binary(add_site, PSK_ADD, *addend, out);
        return out;
    }

    // lower.rs:481-513: x[..., K] · w[K, rest...]
    Tensor dot(const std::string &site, const Tensor &x, const Tensor &w, const Tensor *addend = nullptr, const std::string &add_site = "")
    {
        if (x.axes.empty() || w.axes.empty()) raise(PSK_E7001, "dot: both operands need at least one axis");
        if (x.axes.back().len != w.axes[0].len) raise(PSK_E7001, "dot: contracted axes differ (" + std::to_string(x.axes.back().len) + " vs " + std::to_string(w.axes[0].len) + ")");
        // as an ein over fresh names: the output keeps x's leading axes and w's trailing ones
        std::vector<std::string> xs, ws, os;
        Axes out_axes;
        for (size_t i = 0; i + 1 < x.axes.size(); ++i) { xs.push_back("x" + std::to_string(i)); os.push_back(xs.back()); out_axes.push_back(x.axes[i]); }
        xs.push_back("k");
        ws.push_back("k");
        for (size_t i = 1; i < w.axes.size(); ++i) { ws.push_back("w" + std::to_string(i)); os.push_back(ws.back()); out_axes.push_back(w.axes[i]); }
        Tensor plain;
        if (addend) { plain = *addend; for (auto &a : plain.axes) a.name.clear(); } // aligned by position, as `add` aligns equal shapes
        Tensor out = ein(site, os, {xs, ws}, {&x, &w}, "dot", addend ? &plain : nullptr, add_site);
        out.axes = addend ? addend->axes : out_axes;
        return out;
    }

    // ---- reductions (lower.rs:1221-1255) -----------------------------------------------
    Tensor reduce_axis(const std::string &site, int kind, const std::string &axis, const Tensor &x)
    {
        int p = -1;
        for (size_t i = 0; i < x.axes.size(); ++i) if (x.axes[i].name == axis) { p = (int)i; break; }
        if (p < 0) raise(PSK_E7001, "no axis `" + axis + "` in " + show(x.axes));
        Axes out_axes = x.axes;
        int64_t n = out_axes[p].len;
        out_axes.erase(out_axes.begin() + p);
        int d = site_dtype(site);
        Tensor out = fresh(out_axes, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_REDUCE;
        l.dtype = d;
        l.kind = kind;
        l.iparam[0] = n;
        set_space(l, out_axes, {n});
        std::vector<int> map;
        for (int i = 0, o = 0; i < (int)x.axes.size(); ++i) map.push_back(i == p ? (int)out_axes.size() : o++);
        std::vector<int64_t> st, ss;
        view(x, map, (int)out_axes.size() + 1, st, ss);
        set_operand(l.in[0], x, st, ss);
        set_operand(l.out, out, contiguous(out_axes), {});
        run(l, std::string(kind == PSK_REDUCE_MEAN ? "mean" : "sum") + " axis " + axis, {&x}, out);
        return out;
    }

    Tensor reduce_all(const std::string &site, int kind, const Tensor &x)
    {
        int d = site_dtype(site);
        Tensor out = fresh({}, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_REDUCE;
        l.dtype = d;
        l.kind = kind;
        l.iparam[0] = x.numel();
        // every axis is summed, in row-major order: one summed axis of the whole length
        set_space(l, {}, {x.numel()});
        set_operand(l.in[0], x, {1}, {0});
        set_operand(l.out, out, {}, {});
        run(l, kind == PSK_REDUCE_MEAN ? "mean" : kind == PSK_REDUCE_SUMSQ ? "sum_squares" : "sum", {&x}, out);
        return out;
    }

    // ---- softmax, cross-entropy (lower.rs:1274-1470) -----------------------------------
    Tensor softmax(const std::string &site, const std::string &axis, const Tensor &x, const Tensor *mask)
    {
        int p = -1;
        for (size_t i = 0; i < x.axes.size(); ++i) if (x.axes[i].name == axis) { p = (int)i; break; }
        if (p < 0) raise(PSK_E7001, "no axis `" + axis + "` in " + show(x.axes));
        Axes outer = x.axes;
        int64_t n = outer[p].len;
        outer.erase(outer.begin() + p);
        int d = site_dtype(site);
        Tensor out = fresh(x.axes, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_SOFTMAX;
        l.dtype = d;
        l.masked = mask ? 1 : 0;
        set_space(l, outer, {n});
        std::vector<int> map;
        for (int i = 0, o = 0; i < (int)x.axes.size(); ++i) map.push_back(i == p ? (int)outer.size() : o++);
        std::vector<int64_t> st, ss;
        view(x, map, (int)outer.size() + 1, st, ss);
        set_operand(l.in[0], x, st, ss);
        set_operand(l.out, out, st, {});
        std::vector<const Tensor *> ins = {&x};
        if (mask) {
            std::vector<int> mm, m2;
            if (!align(mask->axes, x.axes, mm)) raise(PSK_E7001, "softmax: the mask " + show(mask->axes) + " does not broadcast into " + show(x.axes));
            for (int q : mm) m2.push_back(map[q]);
            std::vector<int64_t> mst, mss;
            view(*mask, m2, (int)outer.size() + 1, mst, mss);
            set_operand(l.in[1], *mask, mst, mss);
            ins.push_back(mask);
        }
        run(l, "softmax axis " + axis + (mask ? " where" : ""), ins, out);
        return out;
    }

    // The four launches of an attention function as one (PSK_OP_ATTENTION), under the declared order
    // `attention: blockwise`: q [batch, groups, per, seq, hd], k [batch, groups, seq2, hd],
    // v [batch, seq2, groups, hd], result [batch, seq, groups, per, hd] as the last ein would lay it out.
    // `sites`: scores, scaled scores, softmax, result. While magnitudes are being measured the launches
    // stay apart, since the three sites in between are never stored by the fused one.
    Tensor attention_blockwise(const std::vector<std::string> &sites, const Tensor &q, const Tensor &k, const Tensor &v, const Tensor &rt, const Tensor *mask, bool *ran)
    {
        const int64_t B = q.axes[0].len, G = q.axes[1].len, P = q.axes[2].len, T = q.axes[3].len, HD = q.axes[4].len, T2 = k.axes[2].len;
        int d_mid[3];
        for (int i = 0; i < 3; ++i) {
            d_mid[i] = site_dtype(sites[i]);
            if (rz.scaled.count(sites[i])) raise(PSK_E7005, "attention: blockwise: the site " + sites[i] + " is stored in an affine format, which the fused launch never stores");
        }
        int d = site_dtype(sites[3]);
        Axes out_axes = {{"batch", B}, {"seq", T}, {"groups", G}, {"per", P}, {"hd", HD}};
        Tensor out = fresh_at(sites[3], out_axes);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_ATTENTION;
        l.dtype = d;
        l.masked = mask ? 1 : 0;
        l.iparam[0] = rz.online_attention ? 1 : 0;
        l.iparam[1] = d_mid[0]; l.iparam[2] = d_mid[1]; l.iparam[3] = d_mid[2];
        Axes outer = {{"batch", B}, {"groups", G}, {"per", P}, {"seq", T}, {"hd", HD}};
        set_space(l, outer, {T2});
        std::vector<int64_t> st, ss;
        view(q, {0, 1, 2, 3, 4}, 6, st, ss); set_operand(l.in[0], q, st, ss);
        view(k, {0, 1, 5, 4}, 6, st, ss);    set_operand(l.in[1], k, st, ss);
        view(v, {0, 5, 1, 4}, 6, st, ss);    set_operand(l.in[2], v, st, ss);
        set_operand(l.in[3], rt, {}, {});
        std::vector<const Tensor *> ins = {&q, &k, &v, &rt};
        if (mask) {
            if (mask->axes.size() != 2 || mask->axes[0].len != T || mask->axes[1].len != T2) raise(PSK_E7001, "attention: the mask " + show(mask->axes) + " is not over (seq, seq2)");
            view(*mask, {3, 5}, 6, st, ss);
            set_operand(l.in[4], *mask, st, ss);
            ins.push_back(mask);
        }
        view(out, {0, 3, 1, 2, 4}, 6, st, ss);
        set_operand(l.out, out, st, {});
        *ran = run(l, rz.online_attention ? "attention[online]" : "attention[blockwise]", ins, out, true);
        return out;
    }

    Tensor cross_entropy(const std::string &site, const Tensor &logits, const Tensor &y)
    {
        Axes outer = y.axes;
        int64_t v = logits.axes.back().len;
        if (logits.axes.size() != y.axes.size() + 1) raise(PSK_E7001, "cross_entropy: " + show(logits.axes) + " against labels " + show(y.axes));
        int d = site_dtype(site);
        Tensor out = fresh(outer, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_XENT;
        l.dtype = d;
        set_space(l, outer, {v});
        std::vector<int> map;
        for (int i = 0; i < (int)logits.axes.size(); ++i) map.push_back(i);
        std::vector<int64_t> st, ss;
        view(logits, map, (int)outer.size() + 1, st, ss);
        set_operand(l.in[0], logits, st, ss);
        std::vector<int> ym;
        for (int i = 0; i < (int)y.axes.size(); ++i) ym.push_back(i);
        view(y, ym, (int)outer.size() + 1, st, ss);
        set_operand(l.in[1], y, st, ss);
        set_operand(l.out, out, contiguous(outer), {});
        run(l, "cross_entropy", {&logits, &y}, out);
        return out;
    }

    // ---- indexing (lower.rs:1421-1437, 1554-1750) ------------------------------------------
    Tensor embed(const std::string &site, const Tensor &table, const Tensor &ids)
    {
        if (table.axes.size() != 2) raise(PSK_E7001, "embed: the table must have rank 2");
        Axes out_axes = ids.axes;
        out_axes.push_back({"", table.axes[1].len});
        int d = site_dtype(site);
        Tensor out = fresh(out_axes, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_EMBED;
        l.dtype = d;
        l.iparam[0] = table.axes[0].len;
        set_space(l, out_axes, {});
        std::vector<int64_t> ts(out_axes.size(), 0);
        ts[0] = table.axes[1].len; // a row of the table
        if (out_axes.size() > 1) ts[1] = 1; else raise(PSK_E7001, "embed: indices need an axis");
        set_operand(l.in[0], table, ts, {});
        std::vector<int> im;
        for (int i = 0; i < (int)ids.axes.size(); ++i) im.push_back(i);
        std::vector<int64_t> st, ss;
        view(ids, im, (int)out_axes.size(), st, ss);
        set_operand(l.in[1], ids, st, ss);
        set_operand(l.out, out, contiguous(out_axes), {});
        run(l, "embed", {&table, &ids}, out);
        return out;
    }

    // lower.rs:1472-1488: the cotangent of the logits, (softmax - onehot(y)) * ct row by row
    Tensor cross_entropy_vjp(const std::string &site, const Tensor &logits, const Tensor &y, const Tensor &ct)
    {
        if (logits.axes.size() != y.axes.size() + 1 || ct.axes.size() != y.axes.size()) raise(PSK_E7001, "cross_entropy_vjp: " + show(logits.axes) + ", labels " + show(y.axes) + ", cotangent " + show(ct.axes));
        const int64_t v = logits.axes.back().len;
        const int no = (int)y.axes.size();
        int d = site_dtype(site);
        Tensor out = fresh(logits.axes, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_XENT_VJP;
        l.dtype = d;
        set_space(l, y.axes, {v});
        std::vector<int> full, outer;
        for (int i = 0; i <= no; ++i) full.push_back(i);
        for (int i = 0; i < no; ++i) outer.push_back(i);
        std::vector<int64_t> st, ss;
        view(logits, full, no + 1, st, ss);
        set_operand(l.in[0], logits, st, ss);
        view(y, outer, no + 1, st, ss);
        set_operand(l.in[1], y, st, ss);
        view(ct, outer, no + 1, st, ss);
        set_operand(l.in[2], ct, st, ss);
        set_operand(l.out, out, contiguous(logits.axes), {});
        run(l, "cross_entropy_vjp", {&logits, &y, &ct}, out);
        return out;
    }

    // lower.rs:1444-1457: the cotangent of the table: zeros, then one row of ct added per index, in index order
    Tensor embed_vjp(const std::string &site, const Tensor &table, const Tensor &ids, const Tensor &ct)
    {
        if (table.axes.size() != 2 || ct.axes.size() != ids.axes.size() + 1 || ids.axes.empty()) raise(PSK_E7001, "embed_vjp: " + show(table.axes) + ", indices " + show(ids.axes) + ", cotangent " + show(ct.axes));
        int d = site_dtype(site);
        Tensor out = fresh(table.axes, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_EMBED_VJP;
        l.dtype = d;
        l.iparam[0] = table.axes[0].len;
        set_space(l, ct.axes, {});
        const int rank = (int)ct.axes.size();
        std::vector<int64_t> ts(rank, 0);
        ts[0] = table.axes[1].len;
        ts[1] = 1;
        set_operand(l.in[0], table, ts, {});
        std::vector<int> im, cm;
        for (int i = 0; i + 1 < rank; ++i) im.push_back(i);
        for (int i = 0; i < rank; ++i) cm.push_back(i);
        std::vector<int64_t> st, ss;
        view(ids, im, rank, st, ss);
        set_operand(l.in[1], ids, st, ss);
        view(ct, cm, rank, st, ss);
        set_operand(l.in[2], ct, st, ss);
        set_operand(l.out, out, ts, {});
        run(l, "embed_vjp", {&table, &ids, &ct}, out);
        return out;
    }

    // A strided copy of `src` read through `stride`/`off` into `dst` at `dst_off`
    // with `dst_stride`, over `space`.
    void copy_part(const std::string &name, int d, const Axes &space, const Tensor &src, const std::vector<int64_t> &stride, int64_t extra_off, const Tensor &dst, const std::vector<int64_t> &dst_stride, int64_t dst_off, bool count)
    {
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_COPY;
        l.dtype = d;
        set_space(l, space, {});
        set_operand(l.in[0], src, stride, {});
        l.in[0].offset += extra_off;
        set_operand(l.out, dst, dst_stride, {});
        l.out.offset += dst_off;
        int64_t before = launches;
        std::string keep = log;
        run(l, name, {&src}, dst);
        if (!count) { launches = before; log = keep; }
    }

    Tensor slice(const std::string &site, const std::string &axis, int64_t lo, int64_t hi, const Tensor &x)
    {
        int p = -1;
        for (size_t i = 0; i < x.axes.size(); ++i) if (x.axes[i].name == axis) { p = (int)i; break; }
        if (p < 0) raise(PSK_E7001, "no axis `" + axis + "` in " + show(x.axes));
        if (lo > hi || hi > x.axes[p].len) raise(PSK_E7001, "slice " + std::to_string(lo) + ".." + std::to_string(hi) + " outside the axis `" + axis + "`, of length " + std::to_string(x.axes[p].len));
        Axes out_axes = x.axes;
        out_axes[p].len = hi - lo;
        int d = x.is_index ? PSK_I64 : site_dtype(site);
        Tensor out = fresh(out_axes, d, x.is_index, x.bound);
        auto st = x.strides();
        copy_part("slice " + axis + ": " + std::to_string(lo) + ".." + std::to_string(hi), d, out_axes, x, st, lo * st[p], out, contiguous(out_axes), 0, true);
        return out;
    }

    // The same elements without a copy: a view of x (merged launches; the reference's buffers have no strides,
    // so its slice is a nest of its own, lower.rs:1554).
    Tensor slice_view(const std::string &axis, int64_t lo, int64_t hi, const Tensor &x)
    {
        int p = -1;
        for (size_t i = 0; i < x.axes.size(); ++i) if (x.axes[i].name == axis) { p = (int)i; break; }
        if (p < 0 || lo > hi || hi > x.axes[p].len) raise(PSK_E7001, "slice of `" + axis + "` outside " + show(x.axes));
        Tensor v = x;
        v.vstrides = x.strides();
        v.off += lo * v.vstrides[p];
        v.axes[p].len = hi - lo;
        return v;
    }

    // lower.rs:1574-1588: zeros of the template's shape with ct at lo..hi of the axis. One nest in the reference
    // (a zero fill, then the stores); here the host's zeros and one copy, counted as the one launch it is.
    Tensor slice_vjp(const std::string &site, const std::string &axis, int64_t lo, int64_t hi, const Tensor &tmpl, const Tensor &ct)
    {
        int p = -1;
        for (size_t i = 0; i < tmpl.axes.size(); ++i) if (tmpl.axes[i].name == axis) { p = (int)i; break; }
        if (p < 0 || ct.axes.size() != tmpl.axes.size() || ct.axes[p].len != hi - lo || hi > tmpl.axes[p].len)
            raise(PSK_E7001, "slice_vjp " + axis + ": " + std::to_string(lo) + ".." + std::to_string(hi) + ": a cotangent of " + show(ct.axes) + " into " + show(tmpl.axes));
        int d = site_dtype(site);
        const int64_t before = launches;
        Tensor out = zeros(site, tmpl.axes);
        launches = before;
        auto os = contiguous(tmpl.axes);
        copy_part("slice_vjp " + axis + ": " + std::to_string(lo) + ".." + std::to_string(hi), d, ct.axes, ct, ct.strides(), 0, out, os, lo * os[p], true);
        return out;
    }

    Tensor concat(const std::string &site, const std::string &axis, const Tensor &x, const Tensor &y)
    {
        int p = -1;
        for (size_t i = 0; i < x.axes.size(); ++i) if (x.axes[i].name == axis) { p = (int)i; break; }
        bool same = p >= 0 && x.axes.size() == y.axes.size() && y.axes[p].name == axis;
        for (size_t k = 0; same && k < x.axes.size(); ++k) same = (int)k == p || x.axes[k].len == y.axes[k].len;
        if (!same) raise(PSK_E7001, "concat " + axis + ": " + show(x.axes) + " and " + show(y.axes));
        Axes out_axes = x.axes;
        out_axes[p].len += y.axes[p].len;
        int d = site_dtype(site);
        Tensor out = fresh(out_axes, d);
        auto os = contiguous(out_axes);
        // one nest of two loops in the reference (lower.rs:1592); two kernels here, one launch
        const bool was = calibrating;
        calibrating = false; // the output is whole only after the second part
        copy_part("concat " + axis, d, x.axes, x, x.strides(), 0, out, os, 0, true);
        calibrating = was;
        copy_part("concat " + axis, d, y.axes, y, y.strides(), 0, out, os, x.axes[p].len * os[p], false);
        return out;
    }

    // out[lead.., hh, s, d] = in[lead.., s, hh·hd + d] (lower.rs:1614)
    Tensor split_heads(const std::string &site, int64_t h, int64_t hd, const Tensor &x)
    {
        size_t r = x.axes.size();
        if (r < 2 || x.axes[r - 1].len != h * hd) raise(PSK_E7001, "split_heads: expected a trailing axis of length " + std::to_string(h * hd));
        Axes out_axes(x.axes.begin(), x.axes.end() - 2);
        out_axes.push_back({"heads", h});
        out_axes.push_back(x.axes[r - 2]);
        out_axes.push_back({"hd", hd});
        int d = site_dtype(site);
        Tensor out = fresh(out_axes, d);
        auto xs = x.strides();
        std::vector<int64_t> st(xs.begin(), xs.end() - 2);
        st.push_back(hd);        // heads
        st.push_back(xs[r - 2]); // seq
        st.push_back(1);         // hd
        copy_part("split_heads " + std::to_string(h) + "x" + std::to_string(hd), d, out_axes, x, st, 0, out, contiguous(out_axes), 0, true);
        return out;
    }

    // out[lead.., s, hh·hd + d] = in[lead.., hh, s, d] (lower.rs:1639)
    Tensor merge_heads(const std::string &site, int64_t h, int64_t hd, const Tensor &x)
    {
        size_t r = x.axes.size();
        if (r < 3) raise(PSK_E7001, "merge_heads: expected [..., heads, seq, hd]");
        Axes out_axes(x.axes.begin(), x.axes.end() - 3);
        out_axes.push_back(x.axes[r - 2]);
        out_axes.push_back({"model", h * hd});
        int d = site_dtype(site);
        Tensor out = fresh(out_axes, d);
        // iterate (lead.., s, hh, d): the output is contiguous over it
        Axes space(x.axes.begin(), x.axes.end() - 3);
        space.push_back(x.axes[r - 2]);
        space.push_back({"", h});
        space.push_back({"", hd});
        auto xs = x.strides();
        std::vector<int64_t> st(xs.begin(), xs.end() - 3);
        st.push_back(xs[r - 2]);
        st.push_back(xs[r - 3]);
        st.push_back(1);
        copy_part("merge_heads " + std::to_string(h) + "x" + std::to_string(hd), d, space, x, st, 0, out, contiguous(space), 0, true);
        return out;
    }

    Tensor iota(int kind, const std::string &name, const Axes &out_axes, bool is_index, int64_t bound, int d)
    {
        Tensor out = fresh(out_axes, d, is_index, bound);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_IOTA;
        l.kind = kind;
        l.dtype = d;
        set_space(l, out_axes, {});
        set_operand(l.out, out, contiguous(out_axes), {});
        run(l, name, {}, out);
        return out;
    }
    Tensor positions(const std::string &site, const std::string &axis, int64_t n) { return iota(PSK_IOTA_POSITIONS, "positions " + axis, {{axis, n}}, true, n, site_dtype(site)); }
    Tensor causal_mask(const std::string &site, const std::string &axis, int64_t n) { return iota(PSK_IOTA_CAUSAL, "causal_mask " + axis, {{axis, n}, {axis + "2", n}}, true, 2, site_dtype(site)); }

    // ---- retags: split and merge of an axis are the host's (host.rs:1510-1544) ------------
    Tensor split(const Tensor &x, const std::string &axis, const std::vector<Axis> &parts)
    {
        Tensor t = x;
        for (size_t i = 0; i < t.axes.size(); ++i)
            if (t.axes[i].name == axis) {
                int64_t n = 1;
                for (auto &p : parts) n *= p.len;
                if (n != t.axes[i].len) raise(PSK_E7001, "split: the parts of `" + axis + "` do not multiply to its length");
                if (t.q_over >= 0) {
                    // the contracted axis read as several (BufKind::Quant's span, presk-kernel/src/ir.rs:20-30)
                    if ((int)i < t.q_over) t.q_over += (int)parts.size() - 1;
                    else if ((int)i < t.q_over + t.q_span) t.q_span += (int)parts.size() - 1;
                }
                if (!t.vstrides.empty()) {
                    int64_t acc = t.vstrides[i];
                    std::vector<int64_t> ps(parts.size());
                    for (int k = (int)parts.size() - 1; k >= 0; --k) { ps[k] = acc; acc *= parts[k].len; }
                    t.vstrides.erase(t.vstrides.begin() + i);
                    t.vstrides.insert(t.vstrides.begin() + i, ps.begin(), ps.end());
                }
                t.axes.erase(t.axes.begin() + i);
                t.axes.insert(t.axes.begin() + i, parts.begin(), parts.end());
                return t;
            }
        raise(PSK_E7001, "split: no axis `" + axis + "` in " + show(x.axes));
    }
    Tensor merge(const Tensor &x, const std::string &a, const std::string &b)
    {
        Tensor t = x;
        for (size_t i = 0; i + 1 < t.axes.size(); ++i)
            if (t.axes[i].name == a && t.axes[i + 1].name == b) {
                if (!t.vstrides.empty()) {
                    if (t.vstrides[i] != t.vstrides[i + 1] * t.axes[i + 1].len) raise(PSK_E7001, "merge: `" + a + "`, `" + b + "` of a view are not one run of elements");
                    t.vstrides.erase(t.vstrides.begin() + i);
                }
                t.axes[i] = {"", t.axes[i].len * t.axes[i + 1].len};
                t.axes.erase(t.axes.begin() + i + 1);
                return t;
            }
        raise(PSK_E7001, "merge: `" + a + "`, `" + b + "` are not adjacent axes of " + show(x.axes));
    }
    Tensor rename_last(const Tensor &x, const std::string &name)
    {
        Tensor t = x;
        t.axes.back().name = name;
        return t;
    }

    // ---- parameters ---------------------------------------------------------------------------
    const Tensor &param(const std::string &path) const
    {
        auto it = params.find(path);
        if (it == params.end()) raise(PSK_E7001, "the parameter `" + path + "` was not given");
        return it->second;
    }
    // Layer l of a stacked parameter: a view, nothing copied (host.rs:2118-2151).
    Tensor layer(const Tensor &t, int64_t l) const
    {
        Tensor v = t;
        int64_t chunk = t.numel() / t.axes[0].len;
        v.off += l * chunk;
        v.axes.erase(v.axes.begin());
        if (t.q_over >= 0) {
            int64_t klen = 1;
            for (int i = t.q_over; i < t.q_over + t.q_span; ++i) klen *= t.axes[i].len;
            int64_t schunk = chunk / klen;
            v.soff += l * schunk;
            v.q_over -= 1;
        }
        return v;
    }

    int param_dtype(const std::string &path, bool &quant, QuantSpec &qs) const
    {
        quant = false;
        auto q = rz.quant.find(path);
        if (q != rz.quant.end()) { quant = true; qs = q->second; return PSK_I8; }
        auto p = rz.params.find(path);
        if (p != rz.params.end()) return p->second;
        return rz.dflt;
    }

    void store_param(const std::string &path, const Tensor &raw)
    {
        bool quant;
        QuantSpec qs;
        int d = param_dtype(path, quant, qs);
        Tensor t;
        if (quant) {
            int rank = (int)raw.axes.size();
            int over = qs.over < 0 ? rank + qs.over : qs.over;
            if (over < 0 || over >= rank) raise(PSK_E7001, "quant[" + path + "]: no axis " + std::to_string(qs.over));
            int64_t outer = 1, inner = 1, k = raw.axes[over].len;
            for (int i = 0; i < over; ++i) outer *= raw.axes[i].len;
            for (int i = over + 1; i < rank; ++i) inner *= raw.axes[i].len;
            t = fresh(raw.axes, PSK_I8);
            t.dtype = PSK_I8;
            t.scales = std::make_shared<Storage>(vt, (size_t)(outer * inner) * 4);
            t.q_over = over;
            if (!vt->quantize) raise(PSK_E7005, "this executor does not quantise weights");
            check(vt->quantize(vt->self, raw.ptr(), raw.dtype, (int8_t *)t.ptr(), (float *)t.scales->p, outer, k, inner), "quantize");
        } else if (d == raw.dtype) {
            t = raw;
        } else {
            t = fresh(raw.axes, d);
            convert_into(raw, t);
        }
        params[path] = t;
    }

    // ===========================================================================
    // The models. Each function below is one function of the source program.
    // ===========================================================================

    // examples/coverage/llama.psk:34-40. %0 θ, %1 x.
    Tensor llama_rmsnorm(const Tensor &gamma, const Tensor &x)
    {
        const std::string f = "RMSNorm.apply";
        if (rz.merged_launches && rz.order == PSK_ORDER_DEVICE && !calibrating && !x.affine) {
            bool plain = true;
            for (auto site : {"/%2", "/%3", "/%5", "/%7"}) plain = plain && !rz.scaled.count(f + site);
            if (plain) {
                // the four launches below as one, when the executor takes it (PSK_OP_RMSNORM: their bits); the result's
                // own site may be a `scaled` one (the operand of integer-sum projections): its codes are then what the
                // last group's store writes
                Tensor eps = scalar(f + "/%5", 1e-5);
                const int d10 = site_dtype(f + "/%10");
                Tensor out = fresh_at(f + "/%10", x.axes);
                psk_launch l;
                memset(&l, 0, sizeof l);
                l.op = PSK_OP_RMSNORM;
                l.dtype = d10;
                l.iparam[0] = x.axes.back().len;
                l.iparam[1] = rz.dtype_at(f + "/%2"); l.iparam[2] = rz.dtype_at(f + "/%3"); l.iparam[3] = rz.dtype_at(f + "/%7");
                set_space(l, x.axes, {});
                set_operand(l.in[0], x, x.strides(), {});
                set_operand(l.in[1], eps, {}, {});
                std::vector<int> map;
                if (align(gamma.axes, x.axes, map)) {
                    std::vector<int64_t> st, ss;
                    view(gamma, map, (int)x.axes.size(), st, ss);
                    set_operand(l.in[2], gamma, st, ss);
                    set_operand(l.out, out, out.strides(), {});
                    if (run(l, "rmsnorm[merged]", {&x, &eps, &gamma}, out, true)) return out;
                }
            }
        }
        Tensor x2 = binary(f + "/%2", PSK_MUL, x, x);
        Tensor ms = reduce_axis(f + "/%3", PSK_REDUCE_MEAN, "model", x2);
        Tensor eps = scalar(f + "/%5", 1e-5);
        Tensor rt = fused(f + "/%7", {Bn(PSK_ADD, 0, 1), U(PSK_SQRT, S(0))}, {&ms, &eps});
        return fused(f + "/%10", {Bn(PSK_DIV, 0, 1), Bn(PSK_MUL, S(0), 2)}, {&x, &rt, &gamma});
    }

    // llama.psk:55-59
    // examples/spec/rope/rope.psk:33-37, Llama 3's scaling of the frequencies with its defaults:
    // s = clamp((context·ω / 2π − lo) / (hi − lo), 0, 1), ω' = ω · ((1 − s) / k + s); clamp is min(max(x, lo), hi).
    Tensor llama3_scaling(const Tensor &w)
    {
        const std::string f = "llama3_scaling";
        Tensor ctx = scalar(f + "/%6", 8192.0), two_pi = scalar(f + "/%8", 6.283185307179586), lo = scalar(f + "/%10", 1.0), span = scalar(f + "/%12", 4.0 - 1.0);
        Tensor zero = scalar(f + "/%14", 0.0), one = scalar(f + "/%15", 1.0), k = scalar(f + "/%19", 32.0);
        Tensor sc = fused(f + "/%17", {Bn(PSK_MUL, 0, 1), Bn(PSK_DIV, S(0), 2), Bn(PSK_SUB, S(1), 3), Bn(PSK_DIV, S(2), 4), Bn(PSK_MAX, S(3), 5), Bn(PSK_MIN, S(4), 6)},
                          {&ctx, &w, &two_pi, &lo, &span, &zero, &one});
        return fused(f + "/%24", {Bn(PSK_SUB, 0, 1), Bn(PSK_DIV, S(0), 2), Bn(PSK_ADD, S(1), 1), Bn(PSK_MUL, 3, S(2))}, {&one, &sc, &k, &w});
    }

    double rope_base = 1e4; // the base of the frequencies: 10 000 in llama.psk; an entry may set another
    Tensor llama_frequencies()
    {
        const std::string f = "frequencies";
        int64_t hd = C("D") / C("H");
        Tensor two = scalar(f + "/%1", 2.0);
        Tensor neg = unary(f + "/%2", PSK_NEG, two);
        Tensor pos = positions(f + "/%3", "rot", hd / 2);
        Tensor rp = unary(f + "/%4", PSK_REAL, pos);
        Tensor hdr = scalar(f + "/%7", (double)hd);
        Tensor base = scalar(f + "/%10", rope_base);
        Tensor lg = unary(f + "/%11", PSK_LOG, base);
        return fused(f + "/%13", {Bn(PSK_MUL, 0, 1), Bn(PSK_DIV, S(0), 2), Bn(PSK_MUL, S(1), 3), U(PSK_EXP, S(2))}, {&neg, &rp, &hdr, &lg});
    }

    // llama.psk:61-62
    bool rope_llama3 = false;
    Tensor llama_angles(int64_t T)
    {
        const std::string f = "angles";
        Tensor pos = positions(f + "/%0", "seq", T);
        Tensor rp = unary(f + "/%1", PSK_REAL, pos);
        Tensor fr = llama_frequencies();
        if (rope_llama3) fr = llama3_scaling(fr);
        return ein(f + "/%3", {"seq", "rot"}, {{"seq"}, {"rot"}}, {&rp, &fr});
    }

    // llama.psk:66-72. %0 φ, %1 x.
    Tensor llama_rope(const Tensor &phi, const Tensor &x)
    {
        const std::string f = "rope";
        int64_t hd = x.axes.back().len;
        Tensor p = split(x, "hd", {{"pair", 2}, {"rot", hd / 2}});
        if (rz.merged_launches && !calibrating) {
            // The same values from fewer launches: the two slices are views of x, cos and sin of the one angle table
            // are computed once a call, and each half is written where the concatenation would copy it. Every
            // site keeps its type's rounding, so this needs the copies' sites to be of the type they copy.
            const int dx = x.dtype, d9 = rz.dtype_at(f + "/%9"), d12 = rz.dtype_at(f + "/%12");
            bool plain = !x.affine && rz.dtype_at(f + "/%3") == dx && rz.dtype_at(f + "/%4") == dx && d9 == d12 && rz.dtype_at(f + "/%13") == d9;
            for (auto site : {"/%3", "/%4", "/%9", "/%12", "/%13"}) plain = plain && !rz.scaled.count(f + site);
            if (plain) {
                Tensor x0 = slice_view("pair", 0, 1, p), x1 = slice_view("pair", 1, 2, p);
                auto key = std::make_pair(phi.ptr(), phi.off);
                auto hit = rope_tables.find(key);
                if (hit == rope_tables.end()) hit = rope_tables.emplace(key, std::make_pair(unary(f + "/%5", PSK_COS, phi), unary(f + "/%6", PSK_SIN, phi))).first;
                const Tensor &c = hit->second.first, &s = hit->second.second;
                Tensor cat = fresh_at(f + "/%13", p.axes);
                bool one = false;
                if (d9 == dx && c.dtype == dx && s.dtype == dx && !c.affine && !s.affine && p.vstrides.empty()) {
                    // both halves in one launch (PSK_OP_ROPE), when the executor takes it
                    psk_launch l;
                    memset(&l, 0, sizeof l);
                    l.op = PSK_OP_ROPE;
                    l.dtype = site_dtype(f + "/%13");
                    set_space(l, p.axes, {});
                    const int na = (int)p.axes.size();
                    set_operand(l.in[0], p, p.strides(), {});
                    std::vector<int64_t> st(na, 0), ss;
                    st[na - 3] = c.axes[1].len; st[na - 1] = 1;
                    set_operand(l.in[1], c, st, {});
                    set_operand(l.in[2], s, st, {});
                    set_operand(l.out, cat, cat.strides(), {});
                    one = c.axes.size() == 2 && c.axes[0].len == p.axes[na - 3].len && c.axes[1].len == p.axes[na - 1].len
                        && run(l, "rope[merged]", {&p, &c, &s}, cat, true);
                }
                if (!one) {
                    Tensor lo = slice_view("pair", 0, 1, cat), hi = slice_view("pair", 1, 2, cat);
                    fused(f + "/%9", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_SUB, S(0), S(1))}, {&x0, &c, &x1, &s}, "", &lo);
                    fused(f + "/%12", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_ADD, S(0), S(1))}, {&x1, &c, &x0, &s}, "", &hi);
                }
                Tensor m = merge(cat, "pair", "rot");
                m.axes.back().name = "hd";
                return m;
            }
        }
        Tensor x0 = slice(f + "/%3", "pair", 0, 1, p);
        Tensor x1 = slice(f + "/%4", "pair", 1, 2, p);
        Tensor c = unary(f + "/%5", PSK_COS, phi);
        Tensor s = unary(f + "/%6", PSK_SIN, phi);
        Tensor a = fused(f + "/%9", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_SUB, S(0), S(1))}, {&x0, &c, &x1, &s});
        Tensor b = fused(f + "/%12", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_ADD, S(0), S(1))}, {&x1, &c, &x0, &s});
        Tensor cat = concat(f + "/%13", "pair", a, b);
        Tensor m = merge(cat, "pair", "rot");
        m.axes.back().name = "hd";
        return m;
    }

    // ---- generation with a cache of keys and values -------------------------------------------------------
    // The reference's serve loop calls the generation function on the whole window for every new token
    // (crates/presk-serve/src/lib.rs:241: every position's keys and values are computed again). Every launch of
    // the decoder treats the rows of (batch, seq) independently except the attention, which reads the keys and
    // values of the positions before; so the last position's logits need only that position's row through every
    // launch, plus the earlier positions' keys (after `rope`) and values, which do not change. `prefill` runs a
    // window as `apply` does and keeps them, a layer each, in the layouts the attention's contractions read:
    // k [batch, groups, TMAX, hd], v [batch, TMAX, groups, hd]; `step` runs one new position a sequence against
    // them. Under the sequential order `step`'s logits are the bits of the last row of `apply` on the whole
    // window: the same launches on the same numbers in the same order, fewer rows of them.
    enum KvMode { KV_OFF, KV_PREFILL, KV_STEP };
    struct KvCache {
        int64_t batch = 0, tmax = 0, len = 0;
        std::vector<Tensor> k, v;
    } kv;
    KvMode kv_mode = KV_OFF;

    void kv_store(int64_t l, const Tensor &k, const Tensor &v, int64_t at)
    {
        const int64_t B = k.axes[0].len, G = k.axes[1].len, T = k.axes[2].len, HD = k.axes[3].len;
        if (k.affine || v.affine) raise(PSK_E7005, "prefill: keys or values stored in an affine format are not kept");
        if ((int64_t)kv.k.size() <= l) { kv.k.resize(l + 1); kv.v.resize(l + 1); }
        if (!kv.k[l].st) {
            kv.k[l] = fresh({{"batch", B}, {"groups", G}, {"seq2", kv.tmax}, {"hd", HD}}, k.dtype);
            kv.v[l] = fresh({{"batch", B}, {"seq2", kv.tmax}, {"groups", G}, {"hd", HD}}, v.dtype);
        }
        if (kv.k[l].dtype != k.dtype || kv.v[l].dtype != v.dtype || kv.k[l].axes[0].len != B) raise(PSK_E7001, "step: the cache was filled under another batch or another type");
        if (at + T > kv.tmax) raise(PSK_E7001, "the cache holds TMAX = " + std::to_string(kv.tmax) + " positions; position " + std::to_string(at + T - 1) + " does not fit");
        // copies, not launches of the program: the positions' keys and values to their rows of the cache
        copy_part("cache k", k.dtype, k.axes, k, k.strides(), 0, kv.k[l], kv.k[l].strides(), at * HD, false);
        copy_part("cache v", v.dtype, v.axes, v, v.strides(), 0, kv.v[l], kv.v[l].strides(), at * G * HD, false);
    }

    // The first n positions of a layer's cache, as the attention's operands: views, nothing copied.
    Tensor kv_view(const Tensor &c, int64_t n)
    {
        Tensor v = c;
        v.vstrides = c.strides();
        for (auto &a : v.axes)
            if (a.name == "seq2") a.len = n;
        return v;
    }

    // llama.psk:86-110. %0 θ, %1 x, %2 mask, %3 φ.
    Tensor llama_attention(int64_t l, const Tensor &x, const Tensor &mask, const Tensor &phi, const Tensor *residual = nullptr, const std::string &add_site = "")
    {
        const std::string f = "Attention.apply";
        const int64_t D = C("D"), H = C("H"), G = C("G", H), HD = D / H, P = H / G;
        Tensor wq = layer(param("blocks.attn.wq"), l), wk = layer(param("blocks.attn.wk"), l), wv = layer(param("blocks.attn.wv"), l), wo = layer(param("blocks.attn.wo"), l);
        wq.axes = {{"model", D}, {"qout", D}};
        wk.axes = {{"model", D}, {"kvout", G * HD}};
        wv.axes = {{"model", D}, {"kvout", G * HD}};
        wo.axes = {{"headhd", D}, {"model", D}};
        Tensor wq3 = split(split(wq, "qout", {{"groups", G}, {"rest", P * HD}}), "rest", {{"per", P}, {"hd", HD}});
        Tensor qe = ein(f + "/%7", {"batch", "groups", "per", "seq", "hd"}, {{"batch", "seq", "model"}, {"model", "groups", "per", "hd"}}, {&x, &wq3});
        Tensor q = llama_rope(phi, qe);
        Tensor wk3 = split(wk, "kvout", {{"groups", G}, {"hd", HD}});
        Tensor ke = ein(f + "/%11", {"batch", "groups", "seq", "hd"}, {{"batch", "seq", "model"}, {"model", "groups", "hd"}}, {&x, &wk3});
        Tensor k = llama_rope(phi, ke);
        Tensor vd = dot(f + "/%14", x, wv);
        vd.axes.back().name = "kvout";
        Tensor v = split(vd, "kvout", {{"groups", G}, {"hd", HD}});
        const Tensor *use_mask = &mask;
        if (kv_mode == KV_PREFILL) kv_store(l, k, v, 0);
        if (kv_mode == KV_STEP) {
            // the new position's keys and values join the cache; the attention reads every position so far, all
            // of them allowed to the new one (the causal mask's last row), so the softmax needs no mask:
            // with every position allowed the masked nest computes the unmasked one's bits (lower.rs:1368-1419)
            kv_store(l, k, v, kv.len);
            k = kv_view(kv.k[l], kv.len + 1);
            v = kv_view(kv.v[l], kv.len + 1);
            use_mask = nullptr;
        }
        Tensor o;
        bool fused_attention = false;
        Tensor hdr, rt;
        if (rz.blockwise_attention && !calibrating) {
            // the root is computed before the scores here and after them below; neither reads the other
            hdr = scalar(f + "/%18", (double)HD);
            rt = unary(f + "/%19", PSK_SQRT, hdr);
            // (a decode step passes no mask: the executor then streams the cache for the one new position)
            o = attention_blockwise({f + "/%16", f + "/%20", f + "/%21", f + "/%22"}, q, k, v, rt, use_mask, &fused_attention);
        }
        if (!fused_attention) {
            Tensor se = ein(f + "/%16", {"batch", "groups", "per", "seq", "seq2"}, {{"batch", "groups", "per", "seq", "hd"}, {"batch", "groups", "seq2", "hd"}}, {&q, &k});
            if (!rt.st) {
                hdr = scalar(f + "/%18", (double)HD);
                rt = unary(f + "/%19", PSK_SQRT, hdr);
            }
            Tensor s = binary(f + "/%20", PSK_DIV, se, rt);
            Tensor a = softmax(f + "/%21", "seq2", s, use_mask);
            o = ein(f + "/%22", {"batch", "seq", "groups", "per", "hd"}, {{"batch", "groups", "per", "seq", "seq2"}, {"batch", "seq2", "groups", "hd"}}, {&a, &v});
        }
        Tensor w2 = split(split(wo, "headhd", {{"groups", G}, {"rest", P * HD}}), "rest", {{"per", P}, {"hd", HD}});
        return ein(f + "/%26", {"batch", "seq", "model"}, {{"batch", "seq", "groups", "per", "hd"}, {"groups", "per", "hd", "model"}}, {&o, &w2}, "", residual, add_site);
    }

    // llama.psk:43,45-50. silu: %0 x, %1 sigmoid, %2 mul.
    Tensor llama_swiglu(int64_t l, const Tensor &x, const Tensor *residual = nullptr, const std::string &add_site = "")
    {
        const std::string f = "SwiGLU.apply";
        Tensor wg = layer(param("blocks.ff.gate.w"), l), wu = layer(param("blocks.ff.up.w"), l), wd = layer(param("blocks.ff.down.w"), l);
        Tensor g = dot("Dense.apply/%3", x, wg);
        const int ds = rz.dtype_at("silu/%2"), dh = rz.dtype_at(f + "/%7");
        if (rz.merged_launches && !calibrating && (ds == PSK_BF16 || ds == PSK_F32) && ds == dh && g.dtype == ds && !g.affine && !rz.scaled.count("silu/%2")) {
            // silu's group and the product with `up` as one launch: silu's value is rounded to its site's type
            // inside the group (PSK_ROUND), so the product reads what the separate launch would have stored
            Tensor u = dot("Dense.apply/%3", x, wu);
            if (u.dtype == ds && !u.affine) {
                Tensor h = fused(f + "/%7", {U(PSK_SIGMOID, 0), Bn(PSK_MUL, 0, S(0)), U(PSK_ROUND, S(1), ds), Bn(PSK_MUL, S(2), 1)}, {&g, &u});
                return dot("Dense.apply/%3", h, wd, residual, add_site);
            }
            Tensor sg = fused("silu/%2", {U(PSK_SIGMOID, 0), Bn(PSK_MUL, 0, S(0))}, {&g});
            Tensor h = binary(f + "/%7", PSK_MUL, sg, u);
            return dot("Dense.apply/%3", h, wd, residual, add_site);
        }
        Tensor sg = fused("silu/%2", {U(PSK_SIGMOID, 0), Bn(PSK_MUL, 0, S(0))}, {&g});
        Tensor u = dot("Dense.apply/%3", x, wu);
        Tensor h = binary(f + "/%7", PSK_MUL, sg, u);
        return dot("Dense.apply/%3", h, wd, residual, add_site);
    }

    // llama.psk:112-119. %0 θ, %1 x, %2 mask, %3 φ.
    Tensor llama_block(int64_t l, const Tensor &x, const Tensor &mask, const Tensor &phi)
    {
        const std::string f = "Block.apply";
        Tensor n1 = llama_rmsnorm(layer(param("blocks.n1.γ"), l), x);
        // the two residual additions follow a contraction each; the contraction takes them along (see `ein`)
        Tensor x1 = llama_attention(l, n1, mask, phi, &x, f + "/%8");
        Tensor n2 = llama_rmsnorm(layer(param("blocks.n2.γ"), l), x1);
        return llama_swiglu(l, n2, &x1, f + "/%13");
    }

    // llama.psk:121-134. %0 θ, %1 ids.
    Tensor llama_apply(const Tensor &ids)
    {
        const std::string f = "Llama.apply";
        const int64_t T = ids.axes[1].len, L = C("L");
        Tensor mask = causal_mask(f + "/%2", "seq", T);
        Tensor e = embed(f + "/%4", param("tok"), ids);
        e.axes.back().name = "model";
        Tensor phi = llama_angles(T);
        Tensor x = e;
        for (int64_t l = 0; l < L; ++l) x = llama_block(l, x, mask, phi);
        Tensor h = llama_rmsnorm(param("norm.γ"), x);
        Tensor logits = dot(f + "/%11", h, param("head"));
        logits.axes.back().name = "vocab";
        return logits;
    }

    // llama.psk:140-142. %0 θ, %1 batch, %2 x, %3 y.
    Tensor llama_loss(const Tensor &ids, const Tensor &y)
    {
        Tensor logits = llama_apply(ids);
        Tensor ce = cross_entropy("loss/%5", logits, y);
        return reduce_all("loss/%6", PSK_REDUCE_MEAN, ce);
    }

    // `prefill`: `apply` on a window, keeping every layer's keys and values. `step`: one new position a sequence.
    Tensor llama_prefill(const Tensor &ids)
    {
        kv = KvCache();
        kv.batch = ids.axes[0].len;
        kv.tmax = C("TMAX");
        if (ids.axes[1].len > kv.tmax) raise(PSK_E7001, "prefill: the window is longer than TMAX");
        struct Restore { psk_host *h; ~Restore() { h->kv_mode = KV_OFF; } } restore{this};
        kv_mode = KV_PREFILL;
        Tensor logits = llama_apply(ids);
        kv.len = ids.axes[1].len;
        return logits;
    }

    Tensor llama_step(const Tensor &ids)
    {
        if (kv.k.empty()) raise(PSK_E7001, "step: no `prefill` came before");
        if (ids.axes.size() != 2 || ids.axes[1].len != 1 || ids.axes[0].len != kv.batch) raise(PSK_E7001, "step: one new position a sequence of the prefilled batch: ids [batch, 1]");
        if (kv.len + 1 > kv.tmax) raise(PSK_E7001, "step: the cache's TMAX = " + std::to_string(kv.tmax) + " positions are used up");
        const std::string f = "Llama.apply";
        const int64_t L = C("L");
        struct Restore { psk_host *h; ~Restore() { h->kv_mode = KV_OFF; } } restore{this};
        kv_mode = KV_STEP;
        Tensor e = embed(f + "/%4", param("tok"), ids);
        e.axes.back().name = "model";
        // the angles of the new position: the last row of the window's table (a row depends on its position alone)
        Tensor phi = slice_view("seq", kv.len, kv.len + 1, llama_angles(kv.len + 1));
        Tensor none; // no mask: see llama_attention
        Tensor x = e;
        for (int64_t l = 0; l < L; ++l) x = llama_block(l, x, none, phi);
        Tensor h = llama_rmsnorm(param("norm.γ"), x);
        Tensor logits = dot(f + "/%11", h, param("head"));
        logits.axes.back().name = "vocab";
        kv.len += 1;
        return logits;
    }

    // examples/spec/layernorm/layernorm.psk; numbering of
    // presk-core/tests/snapshots/lower__core_minigpt.snap. %0 θ, %1 x, %2 eps.
    Tensor layernorm(const Tensor &gamma, const Tensor &beta, const Tensor &x, double eps_v)
    {
        const std::string f = "LayerNorm.apply";
        Tensor mu = reduce_axis(f + "/%3", PSK_REDUCE_MEAN, "model", x);
        Tensor d2 = fused(f + "/%5", {Bn(PSK_SUB, 0, 1), U(PSK_POW, S(0), 2)}, {&x, &mu});
        Tensor var = reduce_axis(f + "/%6", PSK_REDUCE_MEAN, "model", d2);
        Tensor eps = scalar(f + "/%8", eps_v);
        Tensor sd = fused(f + "/%10", {Bn(PSK_ADD, 0, 1), U(PSK_SQRT, S(0))}, {&var, &eps});
        return fused(f + "/%15", {Bn(PSK_SUB, 0, 1), Bn(PSK_DIV, S(0), 2), Bn(PSK_MUL, S(1), 3), Bn(PSK_ADD, S(2), 4)}, {&x, &mu, &sd, &gamma, &beta});
    }

    // The spec's RMSNorm: `pow 2` where Llama's writes `x * x`. %0 θ, %1 x, %2 eps.
    Tensor rmsnorm_spec(const Tensor &gamma, const Tensor &x, double eps_v)
    {
        const std::string f = "RMSNorm.apply";
        Tensor x2 = unary(f + "/%3", PSK_POW, x, 2);
        Tensor ms = reduce_axis(f + "/%4", PSK_REDUCE_MEAN, "model", x2);
        Tensor eps = scalar(f + "/%5", eps_v);
        Tensor rt = fused(f + "/%7", {Bn(PSK_ADD, 0, 1), U(PSK_SQRT, S(0))}, {&ms, &eps});
        return fused(f + "/%10", {Bn(PSK_DIV, 0, 1), Bn(PSK_MUL, S(0), 2)}, {&x, &rt, &gamma});
    }

    // Linear.apply of the snapshot: %2 w, %3 dot, %4 b, %5 add.
    Tensor linear(const std::string &prefix, const Tensor &x)
    {
        Tensor y = dot("Linear.apply/%3", x, param(prefix + ".w"));
        return binary("Linear.apply/%5", PSK_ADD, y, param(prefix + ".b"));
    }

    // Linear{784,256} · ReLU · Linear{256,10}: %0 θ, %1 x; %3 call, %4 relu, %6 call.
    Tensor mlp_apply(const Tensor &x)
    {
        Tensor h = linear("l1", x);
        Tensor r = unary("MLP.apply/%4", PSK_RELU, h);
        return linear("l2", r);
    }
    Tensor mlp_loss(const Tensor &x, const Tensor &y)
    {
        Tensor logits = mlp_apply(x);
        Tensor ce = cross_entropy("loss/%5", logits, y);
        return reduce_all("loss/%6", PSK_REDUCE_MEAN, ce);
    }


    // ===========================================================================
    // examples/spec/mlp/mlp.psk: `mse` and `mse_grad`, the reverse-mode program that the reference's
    // transformation makes of it (crates/presk-core/tests/snapshots/ad__ad_mlp.snap gives every function
    // and let number below). hidden = 4·D. A gradient is a tree of the parameters' shape: its leaves
    // are left in `results` under the parameters' paths.
    // ===========================================================================
    std::map<std::string, Tensor> results;

    // zeros_like (host.rs:1506): a buffer of zeros of the leaf's shape, made by the host, no launch
    Tensor zeros(const std::string &site, const Axes &axes)
    {
        int d = site_dtype(site);
        Tensor out = fresh(axes, d);
        if (out.numel() <= 4096) {
            std::vector<uint8_t> z((size_t)std::max<int64_t>(1, out.numel()) * elem_bytes(d), 0);
            check(vt->upload(vt->self, out.ptr(), z.data(), z.size()), "zeros_like");
            return out;
        }
        // a large leaf: filled on the executor, not sent from the host (still no launch of the program's)
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_IOTA;
        l.kind = PSK_IOTA_FILL;
        l.dtype = d;
        l.fparam[0] = 0.0;
        Axes flat = {{"", out.numel()}};
        set_space(l, flat, {});
        set_operand(l.out, out, {1}, {});
        const int64_t before = launches;
        const std::string keep = log;
        run(l, "zeros_like", {}, out);
        launches = before;
        log = keep;
        return out;
    }

    // lower.rs:1670-1680: x summed into the shape of `tmpl` (whose axes align into x's), the sum kept in the
    // output buffer; the summed axes in x's order
    Tensor sum_to(const std::string &site, const Tensor &x, const Tensor &tmpl)
    {
        std::vector<int> map;
        if (!align(tmpl.axes, x.axes, map)) raise(PSK_E7001, "sum_to: cannot reduce " + show(x.axes) + " to " + show(tmpl.axes));
        std::vector<int> pos(x.axes.size(), -1); // where each axis of x sits in the launch's space
        for (size_t i = 0; i < map.size(); ++i) pos[map[i]] = (int)i;
        std::vector<int64_t> inner;
        int next = (int)map.size();
        for (size_t a = 0; a < x.axes.size(); ++a)
            if (pos[a] < 0) { pos[a] = next++; inner.push_back(x.axes[a].len); }
        int d = site_dtype(site);
        Tensor out = fresh(tmpl.axes, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_REDUCE;
        l.dtype = d;
        l.kind = PSK_REDUCE_SUM_STORED;
        set_space(l, tmpl.axes, inner);
        std::vector<int64_t> st, ss;
        view(x, pos, next, st, ss);
        set_operand(l.in[0], x, st, ss);
        set_operand(l.out, out, contiguous(tmpl.axes), {});
        run(l, "sum_to", {&x}, out);
        return out;
    }

    struct LinearGrad { Tensor w, b, x; };

    // Linear.apply.bwd: %0 θ, %1 x, %2 ct; %8 sum_to ct, b; %9 zeros_like θ; %11 dot_vjp_l ct, w; %12 dot_vjp_r x, ct;
    // %13 zeros_like θ; %15 add of the two trees, leaf by leaf (w, then b).
    LinearGrad spec_linear_bwd(const std::string &prefix, const Tensor &x, const Tensor &ct)
    {
        const std::string f = "Linear.apply.bwd";
        const Tensor &w = param(prefix + ".w"), &b = param(prefix + ".b");
        Tensor gb = sum_to(f + "/%8", ct, b);
        Tensor zw = zeros(f + "/%9", w.axes);
        // the names of the leading axes of ct, then the two of w
        std::vector<std::string> lead, cts, xs;
        for (size_t i = 0; i + 1 < ct.axes.size(); ++i) lead.push_back("x" + std::to_string(i));
        cts = lead; cts.push_back("out");
        xs = lead; xs.push_back("in");
        std::vector<std::string> gx_axes = lead; gx_axes.push_back("in");
        Tensor gx = ein(f + "/%11", gx_axes, {cts, {"in", "out"}}, {&ct, &w}, "dot_vjp_l");
        for (size_t i = 0; i + 1 < x.axes.size(); ++i) gx.axes[i] = x.axes[i];
        gx.axes.back() = x.axes.back();
        Tensor gw = ein(f + "/%12", {"in", "out"}, {xs, cts}, {&x, &ct}, "dot_vjp_r");
        gw.axes = w.axes;
        Tensor zb = zeros(f + "/%13", b.axes);
        LinearGrad g;
        g.w = binary(f + "/%15", PSK_ADD, zw, gw);
        g.b = binary(f + "/%15", PSK_ADD, gb, zb);
        g.x = gx;
        return g;
    }

    // MLP.apply.fwd: the result and the residuals (%3 before gelu, %4 after)
    Tensor spec_mlp_fwd(const Tensor &x, Tensor *pre, Tensor *post, const std::string &fn)
    {
        Tensor h = linear("l1", x);
        Tensor a = unary(fn + "/%4", PSK_GELU, h);
        if (pre) *pre = h;
        if (post) *post = a;
        return linear("l2", a);
    }

    // mse: %3 ŷ, [%4 sub; %5 pow 2] one group, %6 mean
    Tensor spec_mse(const Tensor &x, const Tensor &y)
    {
        Tensor yh = spec_mlp_fwd(x, nullptr, nullptr, "MLP.apply");
        Tensor sq = fused("mse/%5", {Bn(PSK_SUB, 0, 1), U(PSK_POW, S(0), 2)}, {&yh, &y});
        return reduce_all("mse/%6", PSK_REDUCE_MEAN, sq);
    }

    Tensor spec_mse_grad(const Tensor &x, const Tensor &y)
    {
        // mse_grad.lambda0.grad: %3 nat 1, %4 real: the cotangent of the loss
        Tensor ct = scalar("mse_grad.lambda0.grad/%4", 1.0);
        // mse.fwd: %7 MLP.apply.fwd, %9 sub
        Tensor pre, post;
        Tensor yh = spec_mlp_fwd(x, &pre, &post, "MLP.apply.fwd");
        Tensor diff = binary("mse.fwd/%9", PSK_SUB, yh, y);
        // mse.bwd: %8 mean_vjp ct, x; %10 real 2; [%11 pow 1 %5; %12 mul %10, %11; %13 mul %8, %12]; %15 sum_to %13, %4
        const std::string f = "mse.bwd";
        Tensor shaped = fresh(x.axes, site_dtype(f + "/%8")); // the template's shape only
        Tensor g8 = fused(f + "/%8", {U(PSK_DIV_N, 0, (int)x.numel())}, {&ct}, "mean_vjp", nullptr, &shaped.axes);
        Tensor two = scalar(f + "/%10", 2.0);
        Tensor g13 = fused(f + "/%13", {U(PSK_POW, 0, 1), Bn(PSK_MUL, 1, S(0)), Bn(PSK_MUL, 2, S(1))}, {&diff, &two, &g8});
        Tensor g15 = sum_to(f + "/%15", g13, yh);
        // MLP.apply.bwd: %4, %5 residuals; %8 Linear.apply.bwd(l2, %5, ct); %11 zeros_like θ; [%13 gelu' %4; %14 mul %10, %13];
        // %15 Linear.apply.bwd(l1, x, %14); %18 zeros_like θ; %20 add of the trees (l1.w, l1.b, l2.w, l2.b)
        const std::string m = "MLP.apply.bwd";
        LinearGrad g2 = spec_linear_bwd("l2", post, g15);
        Tensor z1w = zeros(m + "/%11", param("l1.w").axes), z1b = zeros(m + "/%11", param("l1.b").axes);
        Tensor g14 = fused(m + "/%14", {U(PSK_GELU_DERIV, 0), Bn(PSK_MUL, 1, S(0))}, {&pre, &g2.x});
        LinearGrad g1 = spec_linear_bwd("l1", x, g14);
        Tensor z2w = zeros(m + "/%18", param("l2.w").axes), z2b = zeros(m + "/%18", param("l2.b").axes);
        results.clear();
        results["l1.w"] = binary(m + "/%20", PSK_ADD, z1w, g1.w);
        results["l1.b"] = binary(m + "/%20", PSK_ADD, z1b, g1.b);
        results["l2.w"] = binary(m + "/%20", PSK_ADD, g2.w, z2w);
        results["l2.b"] = binary(m + "/%20", PSK_ADD, g2.b, z2b);
        return results["l1.w"];
    }


    // ===========================================================================
    // examples/spec/concat/concat.psk `loss`: slices of an index window, the weights of three projections
    // concatenated for one product, its result cut back into three slices, min, max and clamp element by
    // element, a head, the mean cross-entropy. The sites' numbers are not pinned by a snapshot of the reference
    // (they name where a realization file would put a type, nothing else); the value is (tests/run/concat_loss.snap).
    // ===========================================================================
    Tensor toy_loss(const Tensor &w)
    {
        const int64_t T = w.axes[1].len - 1, D = C("D");
        Tensor ids = slice("inputs/%1", "seq", 0, T, w);
        Tensor tgt = slice("targets/%1", "seq", 1, T + 1, w);
        Tensor x = embed("Toy.apply/%3", param("tok"), ids);
        x.axes.back().name = "model";
        Tensor wq = param("qkv.wq"), wk = param("qkv.wk"), wv = param("qkv.wv");
        for (Tensor *t : {&wq, &wk, &wv}) t->axes = {{"model", D}, {"out", D}};
        Tensor w2 = concat("QKV.apply/%5", "out", wq, wk);
        Tensor w3 = concat("QKV.apply/%7", "out", w2, wv);
        Tensor y = dot("QKV.apply/%8", x, w3);
        y.axes.back().name = "out";
        Tensor q = slice("QKV.apply/%9", "out", 0, D, y), k = slice("QKV.apply/%10", "out", D, 2 * D, y), v = slice("QKV.apply/%11", "out", 2 * D, 3 * D, y);
        // hardtanh(q) = min(max(q, -1), 1); leaky(k) = max(k, k * 0.01); g = hardtanh(q) * leaky(k) + min(v, q)
        Tensor one = scalar("hardtanh/%2", 1.0);
        Tensor neg = unary("hardtanh/%3", PSK_NEG, one);
        Tensor c = scalar("leaky/%2", 0.01);
        Tensor g = fused("Toy.apply/%12", {Bn(PSK_MAX, 0, 3), Bn(PSK_MIN, S(0), 4), Bn(PSK_MUL, 1, 5), Bn(PSK_MAX, 1, S(2)), Bn(PSK_MUL, S(1), S(3)), Bn(PSK_MIN, 2, 0), Bn(PSK_ADD, S(4), S(5))},
                         {&q, &k, &v, &neg, &one, &c});
        Tensor head = param("head");
        head.axes = {{"out", D}, {"vocab", C("V")}};
        Tensor logits = dot("Toy.apply/%14", g, head);
        logits.axes.back().name = "vocab";
        Tensor ce = cross_entropy("loss/%5", logits, tgt);
        return reduce_all("loss/%6", PSK_REDUCE_MEAN, ce);
    }

    // The first operand's and the second's share of a cotangent through max(a, b) (min(a, b): called with the
    // operands exchanged), presk-core/src/ad/rules.rs:115-124: diff = a - b, u = heaviside(diff) (1 where diff > 0),
    // ca = ct * u, cb = ct * (1 - u). diff and u have two readers and are launches of their own; 1 - u has one
    // and joins its product.
    void max_vjp(const std::string &f, const Tensor &a, const Tensor &b, const Tensor &ct, const Tensor &one, Tensor *ca, Tensor *cb)
    {
        Tensor diff = binary(f + "/diff", PSK_SUB, a, b);
        Tensor u = unary(f + "/u", PSK_HEAVISIDE, diff);
        if (ca) *ca = binary(f + "/ca", PSK_MUL, ct, u);
        if (cb) *cb = fused(f + "/cb", {Bn(PSK_SUB, 0, 1), Bn(PSK_MUL, 2, S(0))}, {&one, &u, &ct});
    }

    // examples/spec/concat/concat.psk `loss_grad`: the reverse-mode program of `loss`, built by the rules of
    // presk-core/src/ad/rules.rs (cross_entropy_vjp, dot_vjp_l/r, the max/min rule above, slice_vjp, a concat's
    // cotangent cut into two slices, embed_vjp, mean_vjp), cotangents of a value with several readers added in
    // the reverse of the readers' order. The reference's own list of launches for this program is not pinned
    // by a snapshot (neither the sites' numbers, written here as names, nor its additions of zero trees, left
    // out: x + 0 changes no value but a -0); the gradient's values are (tests/run/concat_loss_grad.snap).
    // Leaves in `results`: tok, head, qkv.wq, qkv.wk, qkv.wv.
    Tensor toy_loss_grad(const Tensor &w)
    {
        const int64_t T = w.axes[1].len - 1, D = C("D");
        const std::string f = "loss_grad";
        // the forward pass, every value the reverse pass reads kept
        Tensor ids = slice("inputs/%1", "seq", 0, T, w);
        Tensor tgt = slice("targets/%1", "seq", 1, T + 1, w);
        Tensor tok = param("tok");
        Tensor x = embed("Toy.apply/%3", tok, ids);
        x.axes.back().name = "model";
        Tensor wq = param("qkv.wq"), wk = param("qkv.wk"), wv = param("qkv.wv");
        for (Tensor *t : {&wq, &wk, &wv}) t->axes = {{"model", D}, {"out", D}};
        Tensor w2 = concat("QKV.apply/%5", "out", wq, wk);
        Tensor w3 = concat("QKV.apply/%7", "out", w2, wv);
        Tensor y = dot("QKV.apply/%8", x, w3);
        y.axes.back().name = "out";
        Tensor q = slice("QKV.apply/%9", "out", 0, D, y), k = slice("QKV.apply/%10", "out", D, 2 * D, y), v = slice("QKV.apply/%11", "out", 2 * D, 3 * D, y);
        Tensor one = scalar("hardtanh/%2", 1.0);
        Tensor neg = unary("hardtanh/%3", PSK_NEG, one);
        Tensor c = scalar("leaky/%2", 0.01);
        Tensor m1 = binary(f + "/hardtanh.max", PSK_MAX, q, neg);
        Tensor ht = binary(f + "/hardtanh.min", PSK_MIN, m1, one);
        Tensor kc = binary(f + "/leaky.mul", PSK_MUL, k, c);
        Tensor lk = binary(f + "/leaky.max", PSK_MAX, k, kc);
        Tensor g = fused(f + "/g", {Bn(PSK_MUL, 0, 1), Bn(PSK_MIN, 2, 3), Bn(PSK_ADD, S(0), S(1))}, {&ht, &lk, &v, &q});
        Tensor head = param("head");
        head.axes = {{"out", D}, {"vocab", C("V")}};
        Tensor logits = dot("Toy.apply/%14", g, head);
        logits.axes.back().name = "vocab";
        Tensor ce = cross_entropy("loss/%5", logits, tgt);
        // the reverse pass
        Tensor ct = scalar(f + "/ct", 1.0);
        Tensor c_ce = fused(f + "/mean_vjp", {U(PSK_DIV_N, 0, (int)ce.numel())}, {&ct}, "mean_vjp", nullptr, &ce.axes);
        Tensor c_logits = cross_entropy_vjp(f + "/cross_entropy_vjp", logits, tgt, c_ce);
        Tensor c_g = ein(f + "/head.dot_vjp_l", {"batch", "seq", "out"}, {{"batch", "seq", "vocab"}, {"out", "vocab"}}, {&c_logits, &head}, "dot_vjp_l");
        Tensor c_head = ein(f + "/head.dot_vjp_r", {"out", "vocab"}, {{"batch", "seq", "out"}, {"batch", "seq", "vocab"}}, {&g, &c_logits}, "dot_vjp_r");
        // g = hardtanh(q) * leaky(k) + min(v, q): the sum hands its cotangent to both terms
        Tensor c_v, c_q2;
        max_vjp(f + "/min", q, v, c_g, one, &c_v, &c_q2); // min(v, q): (a, b) = (q, v); the first operand v takes ct * u
        Tensor c_ht = binary(f + "/mul.l", PSK_MUL, c_g, lk);
        Tensor c_lk = binary(f + "/mul.r", PSK_MUL, c_g, ht);
        Tensor c_k1, c_kc;
        max_vjp(f + "/leaky.max", k, kc, c_lk, one, &c_k1, &c_kc);
        Tensor c_k2 = binary(f + "/leaky.mul", PSK_MUL, c_kc, c);
        Tensor c_k = binary(f + "/k.add", PSK_ADD, c_k1, c_k2);
        Tensor c_m1;
        max_vjp(f + "/hardtanh.min", one, m1, c_ht, one, &c_m1, nullptr); // min(m1, 1): (a, b) = (1, m1); the first operand m1 takes ct * u
        Tensor c_q1;
        max_vjp(f + "/hardtanh.max", q, neg, c_m1, one, &c_q1, nullptr);
        Tensor c_q = binary(f + "/q.add", PSK_ADD, c_q2, c_q1);
        // y's three slices, the last reader first
        Tensor yv = slice_vjp(f + "/slice_vjp.v", "out", 2 * D, 3 * D, y, c_v);
        Tensor yk = slice_vjp(f + "/slice_vjp.k", "out", D, 2 * D, y, c_k);
        Tensor yq = slice_vjp(f + "/slice_vjp.q", "out", 0, D, y, c_q);
        Tensor c_y1 = binary(f + "/y.add", PSK_ADD, yv, yk);
        Tensor c_y = binary(f + "/y.add", PSK_ADD, c_y1, yq);
        Tensor c_x = ein(f + "/qkv.dot_vjp_l", {"batch", "seq", "model"}, {{"batch", "seq", "out"}, {"model", "out"}}, {&c_y, &w3}, "dot_vjp_l");
        Tensor c_w3 = ein(f + "/qkv.dot_vjp_r", {"model", "out"}, {{"batch", "seq", "model"}, {"batch", "seq", "out"}}, {&x, &c_y}, "dot_vjp_r");
        c_w3.axes = {{"model", D}, {"out", 3 * D}};
        Tensor c_w2 = slice(f + "/concat.l", "out", 0, 2 * D, c_w3);
        results.clear();
        results["qkv.wv"] = slice(f + "/concat.r", "out", 2 * D, 3 * D, c_w3);
        results["qkv.wq"] = slice(f + "/concat.l", "out", 0, D, c_w2);
        results["qkv.wk"] = slice(f + "/concat.r", "out", D, 2 * D, c_w2);
        results["head"] = c_head;
        results["tok"] = embed_vjp(f + "/embed_vjp", tok, ids, c_x);
        return results["tok"];
    }

    // ===========================================================================
    // examples/tests/data/stack_grad.psk: a tower of L blocks x + tanh(x·w + b) * scale over a stacked parameter
    // tree (blocks.w [L, D, D], blocks.b [L, D]: the fold reads layer l as a view), the loss mean(y^2), and its
    // gradient through the fold: per block, last first, the rules of presk-core/src/ad/rules.rs (add, mul, tanh:
    // ct * (1 - y*y), sum_to for the bias, dot_vjp_l/r), each layer's leaves placed at l of the stacked gradient.
    // As for `toy`, the reference's list of launches is not pinned by a snapshot; the values are
    // (tests/run/stack_grad.snap).
    // ===========================================================================
    Tensor tower_block(int64_t l, const Tensor &x, const Tensor &scale, Tensor *tanh_out)
    {
        const int64_t D = C("D");
        const std::string f = tanh_out ? "Block.apply.fwd" : "Block.apply";
        Tensor w = layer(param("blocks.w"), l), b = layer(param("blocks.b"), l);
        w.axes = {{"model", D}, {"out", D}};
        b.axes = {{"model", D}};
        Tensor h = dot(f + "/%4", x, w);
        h.axes.back().name = "model";
        if (!tanh_out) return fused(f + "/%8", {Bn(PSK_ADD, 0, 1), U(PSK_TANH, S(0)), Bn(PSK_MUL, S(1), 2), Bn(PSK_ADD, 3, S(2))}, {&h, &b, &scale, &x});
        *tanh_out = fused(f + "/%6", {Bn(PSK_ADD, 0, 1), U(PSK_TANH, S(0))}, {&h, &b}); // read again by the reverse pass
        return fused(f + "/%8", {Bn(PSK_MUL, 0, 1), Bn(PSK_ADD, 2, S(0))}, {tanh_out, &scale, &x});
    }

    Tensor tower_loss(const Tensor &x0, const Tensor &scale)
    {
        Tensor x = x0;
        for (int64_t l = 0; l < C("L"); ++l) x = tower_block(l, x, scale, nullptr);
        Tensor sq = unary("loss/%4", PSK_POW, x, 2);
        return reduce_all("loss/%5", PSK_REDUCE_MEAN, sq);
    }

    Tensor tower_loss_grad(const Tensor &x0, const Tensor &scale)
    {
        const int64_t L = C("L"), D = C("D");
        const std::string f = "loss_grad";
        std::vector<Tensor> xs, ts(L);
        Tensor x = x0;
        for (int64_t l = 0; l < L; ++l) {
            xs.push_back(x);
            x = tower_block(l, x, scale, &ts[l]);
        }
        Tensor ct1 = scalar(f + "/ct", 1.0);
        Tensor c_sq = fused(f + "/mean_vjp", {U(PSK_DIV_N, 0, (int)x.numel())}, {&ct1}, "mean_vjp", nullptr, &x.axes);
        Tensor two = scalar(f + "/two", 2.0), one = scalar(f + "/one", 1.0);
        Tensor ct = fused(f + "/pow", {U(PSK_POW, 0, 1), Bn(PSK_MUL, 1, S(0)), Bn(PSK_MUL, 2, S(1))}, {&x, &two, &c_sq});
        const Tensor &pw = param("blocks.w"), &pb = param("blocks.b");
        Tensor gw = zeros(f + "/blocks.w", pw.axes), gb = zeros(f + "/blocks.b", pb.axes);
        for (int64_t l = L - 1; l >= 0; --l) {
            Tensor w = layer(pw, l), b = layer(pb, l);
            w.axes = {{"model", D}, {"out", D}};
            b.axes = {{"model", D}};
            // through x + t * scale, then tanh: ct * scale * (1 - t * t)
            Tensor c_a = fused(f + "/tanh", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 2), Bn(PSK_SUB, 3, S(1)), Bn(PSK_MUL, S(0), S(2))}, {&ct, &scale, &ts[l], &one});
            Tensor c_b = sum_to(f + "/b", c_a, b);
            Tensor ca = c_a;
            ca.axes.back().name = "out";
            Tensor xin = xs[l];
            xin.axes.back().name = "model";
            Tensor c_x = ein(f + "/dot_vjp_l", {"batch", "model"}, {{"batch", "out"}, {"model", "out"}}, {&ca, &w}, "dot_vjp_l");
            Tensor c_w = ein(f + "/dot_vjp_r", {"model", "out"}, {{"batch", "model"}, {"batch", "out"}}, {&xin, &ca}, "dot_vjp_r");
            ct = binary(f + "/x.add", PSK_ADD, ct, c_x);
            copy_part("scatter_params", c_w.dtype, c_w.axes, c_w, c_w.strides(), 0, gw, contiguous(c_w.axes), l * D * D, true);
            copy_part("scatter_params", c_b.dtype, c_b.axes, c_b, c_b.strides(), 0, gb, contiguous(c_b.axes), l * D, true);
        }
        results.clear();
        results["blocks.w"] = gw;
        results["blocks.b"] = gb;
        return gw;
    }

    // ===========================================================================
    // examples/coverage/llama.psk `loss` in reverse mode (`grad(λ θ. loss(θ, batch))(θ)`): the forward pass with
    // every value the reverse pass reads kept (so no merged launch and no blockwise attention here), then the
    // rules of presk-core/src/ad/rules.rs function by function, last let first: mul, div (∂b = -ct·y/b), sqrt,
    // sigmoid (ct·y·(1 - y)), mean_vjp, sum_to for broadcast operands, the `ein` rule (the cotangent contracted with
    // the other operand), softmax (y·(ct - Σ ct·y)), slice_vjp and the concatenation's two slices in `rope`,
    // dot_vjp_l/r, embed_vjp, cross_entropy_vjp. Cotangents of a value with several readers are added in the
    // reverse of the readers' order. The reference keeps no snapshot of this transformed program: the sites are
    // written as names and the list of launches is this derivation; the values are held against an independent
    // float64 reverse-mode statement of the model in the tests. Leaves in `results` under the parameters' paths
    // (stacked leaves as [L, ...]).
    // ===========================================================================
    struct NormKept { Tensor x, rt, d; };
    Tensor train_norm(const Tensor &gamma, const Tensor &x, NormKept &k)
    {
        const std::string f = "RMSNorm.apply.fwd";
        Tensor x2 = binary(f + "/x2", PSK_MUL, x, x);
        Tensor ms = reduce_axis(f + "/ms", PSK_REDUCE_MEAN, "model", x2);
        Tensor eps = scalar(f + "/eps", 1e-5);
        k.x = x;
        k.rt = fused(f + "/rt", {Bn(PSK_ADD, 0, 1), U(PSK_SQRT, S(0))}, {&ms, &eps});
        k.d = binary(f + "/d", PSK_DIV, x, k.rt);
        return binary(f + "/y", PSK_MUL, k.d, gamma);
    }
    Tensor train_norm_bwd(const Tensor &gamma, const NormKept &k, const Tensor &ct, Tensor *c_gamma)
    {
        const std::string f = "RMSNorm.apply.bwd";
        Tensor c_d = binary(f + "/c_d", PSK_MUL, ct, gamma);
        Tensor t = binary(f + "/ct_d", PSK_MUL, ct, k.d);
        *c_gamma = sum_to(f + "/c_gamma", t, gamma);
        Tensor c_x1 = binary(f + "/c_x.div", PSK_DIV, c_d, k.rt);
        Tensor t2 = fused(f + "/c_rt.full", {Bn(PSK_MUL, 0, 1), Bn(PSK_DIV, S(0), 2), U(PSK_NEG, S(1))}, {&c_d, &k.d, &k.rt});
        Tensor c_rt = sum_to(f + "/c_rt", t2, k.rt);
        Tensor two = scalar(f + "/two", 2.0);
        Tensor c_ms = fused(f + "/c_ms", {Bn(PSK_MUL, 0, 1), Bn(PSK_DIV, 2, S(0))}, {&two, &k.rt, &c_rt});
        Tensor c_xx = fused(f + "/mean_vjp", {U(PSK_DIV_N, 0, (int)k.x.axes.back().len)}, {&c_ms}, "mean_vjp", nullptr, &k.x.axes);
        return fused(f + "/c_x", {Bn(PSK_MUL, 0, 1), Bn(PSK_ADD, 2, S(0)), Bn(PSK_ADD, S(1), S(0))}, {&c_xx, &k.x, &c_x1});
    }

    struct RopeKept { Tensor c, s; };
    Tensor train_rope(const Tensor &phi, const Tensor &x, RopeKept &k)
    {
        const std::string f = "rope.fwd";
        const int64_t hd = x.axes.back().len;
        Tensor p = split(x, "hd", {{"pair", 2}, {"rot", hd / 2}});
        Tensor x0 = slice(f + "/x0", "pair", 0, 1, p), x1 = slice(f + "/x1", "pair", 1, 2, p);
        if (!k.c.st) { k.c = unary(f + "/cos", PSK_COS, phi); k.s = unary(f + "/sin", PSK_SIN, phi); }
        Tensor a = fused(f + "/a", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_SUB, S(0), S(1))}, {&x0, &k.c, &x1, &k.s});
        Tensor b = fused(f + "/b", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_ADD, S(0), S(1))}, {&x1, &k.c, &x0, &k.s});
        Tensor m = merge(concat(f + "/cat", "pair", a, b), "pair", "rot");
        m.axes.back().name = "hd";
        return m;
    }
    // The rotation is linear in x: the cotangent goes back through the transposed rotation.
    Tensor train_rope_bwd(const RopeKept &k, const Tensor &ct)
    {
        const std::string f = "rope.bwd";
        const int64_t hd = ct.axes.back().len;
        Tensor cp = split(ct, "hd", {{"pair", 2}, {"rot", hd / 2}});
        Tensor c_a = slice(f + "/c_a", "pair", 0, 1, cp), c_b = slice(f + "/c_b", "pair", 1, 2, cp);
        Tensor c_x0 = fused(f + "/c_x0", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_ADD, S(0), S(1))}, {&c_b, &k.s, &c_a, &k.c});
        Tensor c_x1 = fused(f + "/c_x1", {Bn(PSK_MUL, 0, 1), U(PSK_NEG, 2), Bn(PSK_MUL, S(1), 3), Bn(PSK_ADD, S(0), S(2))}, {&c_b, &k.c, &c_a, &k.s});
        Tensor p1 = slice_vjp(f + "/slice_vjp.x1", "pair", 1, 2, cp, c_x1), p0 = slice_vjp(f + "/slice_vjp.x0", "pair", 0, 1, cp, c_x0);
        Tensor m = merge(binary(f + "/c_p", PSK_ADD, p1, p0), "pair", "rot");
        m.axes.back().name = "hd";
        return m;
    }

    struct AttnKept { Tensor x, q, k, v, a, o; };
    struct AttnGrad { Tensor x, wq, wk, wv, wo; };
    Tensor train_attention(int64_t l, const Tensor &x, const Tensor &mask, const Tensor &phi, RopeKept &rk, AttnKept &kept)
    {
        const std::string f = "Attention.apply.fwd";
        const int64_t D = C("D"), H = C("H"), G = C("G", H), HD = D / H, P = H / G;
        Tensor wq = layer(param("blocks.attn.wq"), l), wk = layer(param("blocks.attn.wk"), l), wv = layer(param("blocks.attn.wv"), l), wo = layer(param("blocks.attn.wo"), l);
        wq.axes = {{"model", D}, {"groups", G}, {"per", P}, {"hd", HD}};
        wk.axes = {{"model", D}, {"groups", G}, {"hd", HD}};
        wv.axes = {{"model", D}, {"kvout", G * HD}};
        wo.axes = {{"groups", G}, {"per", P}, {"hd", HD}, {"model", D}};
        kept.x = x;
        kept.q = train_rope(phi, ein(f + "/q", {"batch", "groups", "per", "seq", "hd"}, {{"batch", "seq", "model"}, {"model", "groups", "per", "hd"}}, {&x, &wq}), rk);
        kept.k = train_rope(phi, ein(f + "/k", {"batch", "groups", "seq", "hd"}, {{"batch", "seq", "model"}, {"model", "groups", "hd"}}, {&x, &wk}), rk);
        Tensor vd = dot(f + "/v", x, wv);
        vd.axes.back().name = "kvout";
        kept.v = split(vd, "kvout", {{"groups", G}, {"hd", HD}});
        Tensor se = ein(f + "/scores", {"batch", "groups", "per", "seq", "seq2"}, {{"batch", "groups", "per", "seq", "hd"}, {"batch", "groups", "seq2", "hd"}}, {&kept.q, &kept.k});
        Tensor rt = unary(f + "/rt", PSK_SQRT, scalar(f + "/hd", (double)HD));
        Tensor sc = binary(f + "/scaled", PSK_DIV, se, rt);
        kept.a = softmax(f + "/softmax", "seq2", sc, &mask);
        kept.o = ein(f + "/o", {"batch", "seq", "groups", "per", "hd"}, {{"batch", "groups", "per", "seq", "seq2"}, {"batch", "seq2", "groups", "hd"}}, {&kept.a, &kept.v});
        return ein(f + "/out", {"batch", "seq", "model"}, {{"batch", "seq", "groups", "per", "hd"}, {"groups", "per", "hd", "model"}}, {&kept.o, &wo});
    }
    AttnGrad train_attention_bwd(int64_t l, const AttnKept &kept, const RopeKept &rk, const Tensor &ct)
    {
        const std::string f = "Attention.apply.bwd";
        const int64_t D = C("D"), H = C("H"), G = C("G", H), HD = D / H, P = H / G;
        Tensor wq = layer(param("blocks.attn.wq"), l), wk = layer(param("blocks.attn.wk"), l), wv = layer(param("blocks.attn.wv"), l), wo = layer(param("blocks.attn.wo"), l);
        wq.axes = {{"model", D}, {"groups", G}, {"per", P}, {"hd", HD}};
        wk.axes = {{"model", D}, {"groups", G}, {"hd", HD}};
        wv.axes = {{"model", D}, {"kvout", G * HD}};
        wo.axes = {{"groups", G}, {"per", P}, {"hd", HD}, {"model", D}};
        AttnGrad g;
        // the output projection, an `ein` of o and wo: each operand's cotangent is ct contracted with the other
        Tensor c_o = ein(f + "/c_o", {"batch", "seq", "groups", "per", "hd"}, {{"batch", "seq", "model"}, {"groups", "per", "hd", "model"}}, {&ct, &wo});
        g.wo = ein(f + "/c_wo", {"groups", "per", "hd", "model"}, {{"batch", "seq", "groups", "per", "hd"}, {"batch", "seq", "model"}}, {&kept.o, &ct});
        Tensor c_a = ein(f + "/c_a", {"batch", "groups", "per", "seq", "seq2"}, {{"batch", "seq", "groups", "per", "hd"}, {"batch", "seq2", "groups", "hd"}}, {&c_o, &kept.v});
        Tensor c_v = ein(f + "/c_v", {"batch", "seq2", "groups", "hd"}, {{"batch", "groups", "per", "seq", "seq2"}, {"batch", "seq", "groups", "per", "hd"}}, {&kept.a, &c_o});
        // softmax: y · (ct - Σ_seq2 ct · y); refused positions have y = 0
        Tensor t = binary(f + "/ct_y", PSK_MUL, c_a, kept.a);
        Tensor sum = reduce_axis(f + "/sum", PSK_REDUCE_SUM, "seq2", t);
        Tensor c_sc = fused(f + "/c_scaled", {Bn(PSK_SUB, 0, 1), Bn(PSK_MUL, 2, S(0))}, {&c_a, &sum, &kept.a});
        Tensor rt = unary(f + "/rt", PSK_SQRT, scalar(f + "/hd", (double)HD));
        Tensor c_se = binary(f + "/c_scores", PSK_DIV, c_sc, rt);
        Tensor c_q = ein(f + "/c_q", {"batch", "groups", "per", "seq", "hd"}, {{"batch", "groups", "per", "seq", "seq2"}, {"batch", "groups", "seq2", "hd"}}, {&c_se, &kept.k});
        Tensor c_k = ein(f + "/c_k", {"batch", "groups", "seq2", "hd"}, {{"batch", "groups", "per", "seq", "seq2"}, {"batch", "groups", "per", "seq", "hd"}}, {&c_se, &kept.q});
        c_k.axes[2].name = "seq";
        // The projections' cotangents with the positions before the heads again ([batch, seq, out]: a copy, no value
        // changes), so that both of a projection's gradients are plain matrix products over rows of (batch, seq).
        auto rows_of = [&](const std::string &site, const Tensor &t, const std::string &out_name) {
            const int r = (int)t.axes.size(); // [batch, heads.., seq, hd]
            Axes oa;
            std::vector<int64_t> st;
            auto ts = t.strides();
            oa.push_back(t.axes[0]); st.push_back(ts[0]);
            oa.push_back(t.axes[r - 2]); st.push_back(ts[r - 2]);
            for (int i = 1; i < r - 2; ++i) { oa.push_back(t.axes[i]); st.push_back(ts[i]); }
            oa.push_back(t.axes[r - 1]); st.push_back(ts[r - 1]);
            Tensor out = fresh(oa, site_dtype(site));
            copy_part("seq_before_heads", out.dtype, oa, t, st, 0, out, contiguous(oa), 0, true);
            int64_t width = 1;
            for (int i = 2; i < r; ++i) width *= oa[i].len;
            out.axes = {oa[0], oa[1], {out_name, width}};
            return out;
        };
        Tensor c_qh = rows_of(f + "/c_q.rows", train_rope_bwd(rk, c_q), "qout"), c_kh = rows_of(f + "/c_k.rows", train_rope_bwd(rk, c_k), "kvout");
        Tensor wq2 = wq, wk2 = wk;
        wq2.axes = {{"model", D}, {"qout", D}};
        wk2.axes = {{"model", D}, {"kvout", G * HD}};
        // v = split(x · wv)
        Tensor c_vd = merge(c_v, "groups", "hd");
        c_vd.axes[1].name = "seq";
        c_vd.axes.back().name = "kvout";
        Tensor cx_v = ein(f + "/v.dot_vjp_l", {"batch", "seq", "model"}, {{"batch", "seq", "kvout"}, {"model", "kvout"}}, {&c_vd, &wv}, "dot_vjp_l");
        g.wv = ein(f + "/v.dot_vjp_r", {"model", "kvout"}, {{"batch", "seq", "model"}, {"batch", "seq", "kvout"}}, {&kept.x, &c_vd}, "dot_vjp_r");
        Tensor cx_k = ein(f + "/cx_k", {"batch", "seq", "model"}, {{"batch", "seq", "kvout"}, {"model", "kvout"}}, {&c_kh, &wk2});
        g.wk = ein(f + "/c_wk", {"model", "kvout"}, {{"batch", "seq", "model"}, {"batch", "seq", "kvout"}}, {&kept.x, &c_kh});
        Tensor cx_q = ein(f + "/cx_q", {"batch", "seq", "model"}, {{"batch", "seq", "qout"}, {"model", "qout"}}, {&c_qh, &wq2});
        g.wq = ein(f + "/c_wq", {"model", "qout"}, {{"batch", "seq", "model"}, {"batch", "seq", "qout"}}, {&kept.x, &c_qh});
        // x is read by q, k, v in that order: the last reader's share first
        g.x = fused(f + "/c_x", {Bn(PSK_ADD, 0, 1), Bn(PSK_ADD, S(0), 2)}, {&cx_v, &cx_k, &cx_q});
        return g;
    }

    struct FfKept { Tensor x, g, sig, sg, u, h; };
    struct FfGrad { Tensor x, gate, up, down; };
    Tensor train_swiglu(int64_t l, const Tensor &x, FfKept &k)
    {
        const std::string f = "SwiGLU.apply.fwd";
        Tensor wg = layer(param("blocks.ff.gate.w"), l), wu = layer(param("blocks.ff.up.w"), l), wd = layer(param("blocks.ff.down.w"), l);
        k.x = x;
        k.g = dot(f + "/gate", x, wg);
        k.sig = unary(f + "/sigmoid", PSK_SIGMOID, k.g);
        k.sg = binary(f + "/silu", PSK_MUL, k.g, k.sig);
        k.u = dot(f + "/up", x, wu);
        k.h = binary(f + "/h", PSK_MUL, k.sg, k.u);
        Tensor y = dot(f + "/down", k.h, wd);
        y.axes.back().name = "model";
        return y;
    }
    FfGrad train_swiglu_bwd(int64_t l, const FfKept &k, const Tensor &ct)
    {
        const std::string f = "SwiGLU.apply.bwd";
        const int64_t D = C("D"), FF = C("FF");
        Tensor wg = layer(param("blocks.ff.gate.w"), l), wu = layer(param("blocks.ff.up.w"), l), wd = layer(param("blocks.ff.down.w"), l);
        wg.axes = {{"model", D}, {"ff", FF}};
        wu.axes = {{"model", D}, {"ff", FF}};
        wd.axes = {{"ff", FF}, {"model", D}};
        const std::vector<std::string> xm = {"batch", "seq", "model"}, xf = {"batch", "seq", "ff"};
        FfGrad g;
        Tensor c_h = ein(f + "/down.dot_vjp_l", xf, {xm, {"ff", "model"}}, {&ct, &wd}, "dot_vjp_l");
        g.down = ein(f + "/down.dot_vjp_r", {"ff", "model"}, {xf, xm}, {&k.h, &ct}, "dot_vjp_r");
        Tensor c_sg = binary(f + "/c_silu", PSK_MUL, c_h, k.u);
        Tensor c_u = binary(f + "/c_up", PSK_MUL, c_h, k.sg);
        // silu(g) = g · σ(g): ct · σ + (ct · g) · σ · (1 - σ)
        Tensor one = scalar(f + "/one", 1.0);
        Tensor c_g = fused(f + "/c_gate", {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 0, 2), Bn(PSK_SUB, 3, 1), Bn(PSK_MUL, 1, S(2)), Bn(PSK_MUL, S(1), S(3)), Bn(PSK_ADD, S(0), S(4))}, {&c_sg, &k.sig, &k.g, &one});
        Tensor cx_u = ein(f + "/up.dot_vjp_l", xm, {xf, {"model", "ff"}}, {&c_u, &wu}, "dot_vjp_l");
        g.up = ein(f + "/up.dot_vjp_r", {"model", "ff"}, {xm, xf}, {&k.x, &c_u}, "dot_vjp_r");
        Tensor cx_g = ein(f + "/gate.dot_vjp_l", xm, {xf, {"model", "ff"}}, {&c_g, &wg}, "dot_vjp_l");
        g.gate = ein(f + "/gate.dot_vjp_r", {"model", "ff"}, {xm, xf}, {&k.x, &c_g}, "dot_vjp_r");
        g.x = binary(f + "/c_x", PSK_ADD, cx_u, cx_g);
        return g;
    }

    Tensor llama_loss_grad(const Tensor &ids, const Tensor &y)
    {
        const std::string f = "loss_grad";
        const int64_t T = ids.axes[1].len, L = C("L");
        Tensor mask = causal_mask("Llama.apply/%2", "seq", T);
        Tensor tok = param("tok");
        Tensor x = embed("Llama.apply/%4", tok, ids);
        x.axes.back().name = "model";
        Tensor phi = llama_angles(T);
        struct BlockKept { Tensor x, x1; NormKept n1, n2; AttnKept at; FfKept ff; };
        std::vector<BlockKept> kept(L);
        RopeKept rk;
        for (int64_t l = 0; l < L; ++l) {
            BlockKept &b = kept[l];
            b.x = x;
            Tensor h1 = train_norm(layer(param("blocks.n1.γ"), l), x, b.n1);
            b.x1 = binary("Block.apply.fwd/x1", PSK_ADD, x, train_attention(l, h1, mask, phi, rk, b.at));
            Tensor h2 = train_norm(layer(param("blocks.n2.γ"), l), b.x1, b.n2);
            x = binary("Block.apply.fwd/x2", PSK_ADD, b.x1, train_swiglu(l, h2, b.ff));
        }
        NormKept nf;
        Tensor hn = train_norm(param("norm.γ"), x, nf);
        Tensor head = param("head");
        head.axes = {{"model", C("D")}, {"vocab", C("V")}};
        Tensor logits = dot("Llama.apply/%11", hn, head);
        logits.axes.back().name = "vocab";
        Tensor ce = cross_entropy("loss/%5", logits, y);
        // the reverse pass
        Tensor ct1 = scalar(f + "/ct", 1.0);
        Tensor c_ce = fused(f + "/mean_vjp", {U(PSK_DIV_N, 0, (int)ce.numel())}, {&ct1}, "mean_vjp", nullptr, &ce.axes);
        Tensor c_logits = cross_entropy_vjp(f + "/cross_entropy_vjp", logits, y, c_ce);
        const std::vector<std::string> xm = {"batch", "seq", "model"}, xv = {"batch", "seq", "vocab"};
        Tensor c_hn = ein(f + "/head.dot_vjp_l", xm, {xv, {"model", "vocab"}}, {&c_logits, &head}, "dot_vjp_l");
        std::map<std::string, Tensor> out;
        out["head"] = ein(f + "/head.dot_vjp_r", {"model", "vocab"}, {xm, xv}, {&hn, &c_logits}, "dot_vjp_r");
        Tensor ct = train_norm_bwd(param("norm.γ"), nf, c_hn, &out["norm.γ"]);
        static const char *stacked[] = {"blocks.n1.γ", "blocks.n2.γ", "blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w"};
        for (auto path : stacked) out[path] = zeros(f + "/" + path, param(path).axes);
        auto place = [&](const char *path, int64_t l, const Tensor &leaf) {
            Tensor &dst = out[path];
            const int64_t chunk = dst.numel() / dst.axes[0].len;
            if (leaf.numel() != chunk) raise(PSK_E10001, std::string("loss_grad: the leaf of `") + path + "` has " + std::to_string(leaf.numel()) + " elements");
            copy_part("scatter_params", leaf.dtype, leaf.axes, leaf, leaf.strides(), 0, dst, contiguous(leaf.axes), l * chunk, true);
        };
        for (int64_t l = L - 1; l >= 0; --l) {
            BlockKept &b = kept[l];
            // x2 = x1 + ff(n2(x1)); x1 = x + attn(n1(x))
            FfGrad fg = train_swiglu_bwd(l, b.ff, ct);
            Tensor c_n2;
            Tensor c_x1 = binary("Block.apply.bwd/c_x1", PSK_ADD, ct, train_norm_bwd(layer(param("blocks.n2.γ"), l), b.n2, fg.x, &c_n2));
            AttnGrad ag = train_attention_bwd(l, b.at, rk, c_x1);
            Tensor c_n1;
            ct = binary("Block.apply.bwd/c_x", PSK_ADD, c_x1, train_norm_bwd(layer(param("blocks.n1.γ"), l), b.n1, ag.x, &c_n1));
            place("blocks.ff.gate.w", l, fg.gate); place("blocks.ff.up.w", l, fg.up); place("blocks.ff.down.w", l, fg.down);
            place("blocks.n2.γ", l, c_n2); place("blocks.n1.γ", l, c_n1);
            place("blocks.attn.wq", l, ag.wq); place("blocks.attn.wk", l, ag.wk); place("blocks.attn.wv", l, ag.wv); place("blocks.attn.wo", l, ag.wo);
            b = BlockKept(); // this block's kept values are no longer read
        }
        out["tok"] = embed_vjp(f + "/embed_vjp", tok, ids, ct);
        results = out;
        return results["tok"];
    }

    // ===========================================================================
    // The optimizer of a training run: `adamw.init`, `adamw.lr`, `adamw.step` as presk-core/src/lower/optim.rs:118-330
    // builds them (AdamW with decoupled decay; schedules constant, linear(warmup), cosine(warmup) written with relu
    // so that they are ordinary primitives). Lets of a parameter tree's type run leaf by leaf; the groups are those
    // fusion.rs forms over the builder's lets: per step two scalar `sub`s (1 - β), the two bias corrections as
    // groups of four scalar steps (1 - exp(t · ln β)), the schedule as one scalar group, and per leaf three groups:
    // m' (3 steps), v' (4 steps), θ' (9 steps). Sites: `adamw.step/%N`, N the root let's number in the builder's
    // order (parameters %0-%4, then every let; a `grad_clip` puts 14 lets before the rest). With `grad_clip = c` the
    // gradient is scaled by min(1, c / (‖g‖₂ + 1e-6)) first: `sum_squares` a leaf, the leaves' sums added by the host
    // in f64 (presk-kernel/src/host.rs:1571-1587; here in the order of the parameters' paths), one scalar group of
    // six steps for the factor, one `mul` a leaf.
    // ===========================================================================
    struct AdamW { double lr = 1e-3, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, weight_decay = 0.0, grad_clip = 0.0; bool clip = false; int schedule = 0; int64_t warmup = 0; } adamw;
    std::map<std::string, Tensor> moment_m, moment_v;

    void adamw_configure(const std::string &text)
    {
        adamw = AdamW();
        moment_m.clear();
        moment_v.clear();
        std::istringstream ss(text);
        std::string tok;
        while (ss >> tok) {
            size_t eq = tok.find('=');
            if (eq == std::string::npos) raise(PSK_E7001, "a hyperparameter is NAME=VALUE, not `" + tok + "`");
            const std::string k = tok.substr(0, eq), v = tok.substr(eq + 1);
            if (k == "lr") adamw.lr = strtod(v.c_str(), nullptr);
            else if (k == "beta1") adamw.beta1 = strtod(v.c_str(), nullptr);
            else if (k == "beta2") adamw.beta2 = strtod(v.c_str(), nullptr);
            else if (k == "eps") adamw.eps = strtod(v.c_str(), nullptr);
            else if (k == "weight_decay") adamw.weight_decay = strtod(v.c_str(), nullptr);
            else if (k == "warmup") adamw.warmup = strtoll(v.c_str(), nullptr, 10);
            else if (k == "schedule") {
                if (v == "constant") adamw.schedule = 0;
                else if (v == "linear") adamw.schedule = 1;
                else if (v == "cosine") adamw.schedule = 2;
                else raise(PSK_E7001, "schedule is constant, linear or cosine, not `" + v + "`");
            } else if (k == "grad_clip") { adamw.grad_clip = strtod(v.c_str(), nullptr); adamw.clip = true; }
            else raise(PSK_E7001, "adamw has no hyperparameter `" + k + "`");
        }
    }

    // adamw.lr(t, total), optim.rs:279-328
    Tensor adamw_lr(int64_t t, int64_t total)
    {
        const std::string f = "adamw.lr";
        Tensor base = scalar(f + "/base", adamw.lr);
        if (adamw.schedule == 0) return base;
        Tensor tr = scalar(f + "/t", (double)t), totr = scalar(f + "/total", (double)total), w = scalar(f + "/warmup", (double)adamw.warmup);
        Tensor one = scalar(f + "/one", 1.0), half = scalar(f + "/half", 0.5), pi = scalar(f + "/pi", 3.14159265358979323846);
        std::vector<StepSpec> st;
        int warm;
        if (adamw.warmup == 0) warm = 3; // the input `one`
        else {
            st.push_back(Bn(PSK_DIV, 1, 2));                          // t / w
            st.push_back(Bn(PSK_SUB, 3, S(0)));                       // min(1, x) = 1 - relu(1 - x)
            st.push_back(U(PSK_RELU, S(1)));
            st.push_back(Bn(PSK_SUB, 3, S(2)));
            warm = S(3);
        }
        const int o = (int)st.size();
        st.push_back(Bn(PSK_SUB, 1, 2));                              // o+0: t - w
        st.push_back(Bn(PSK_SUB, 4, 2));                              // o+1: total - w
        st.push_back(Bn(PSK_SUB, S(o + 1), 3));                       // o+2: ... - 1
        st.push_back(U(PSK_RELU, S(o + 2)));                          // o+3
        st.push_back(Bn(PSK_ADD, S(o + 3), 3));                       // o+4: max(total - w, 1)
        st.push_back(Bn(PSK_DIV, S(o), S(o + 4)));                    // o+5
        st.push_back(U(PSK_RELU, S(o + 5)));                          // o+6
        st.push_back(Bn(PSK_SUB, 3, S(o + 6)));                       // o+7: min(1, .)
        st.push_back(U(PSK_RELU, S(o + 7)));                          // o+8
        st.push_back(Bn(PSK_SUB, 3, S(o + 8)));                       // o+9: the progress p
        int decay;
        if (adamw.schedule == 2) {
            st.push_back(Bn(PSK_MUL, 5, S(o + 9)));                   // o+10: π p
            st.push_back(U(PSK_COS, S(o + 10)));                      // o+11
            st.push_back(Bn(PSK_ADD, 3, S(o + 11)));                  // o+12: 1 + cos
            st.push_back(Bn(PSK_MUL, S(o + 12), 6));                  // o+13: half of it
            decay = S(o + 13);
        } else {
            st.push_back(Bn(PSK_SUB, 3, S(o + 9)));                   // o+10: 1 - p
            decay = S(o + 10);
        }
        st.push_back(Bn(PSK_MUL, warm, decay));
        st.push_back(Bn(PSK_MUL, 0, S((int)st.size() - 1)));
        return fused(f + "/lr", st, {&base, &tr, &w, &one, &totr, &pi, &half});
    }

    // adamw.step(θ, (m, v), g, t, total), optim.rs:156-219; g = the leaves of the last gradient (`results`).
    // θ', m', v' replace the host's parameters and moments; `results` then holds θ' under the parameters'
    // paths and the moments under "m:" + path, "v:" + path.
    void adamw_step(int64_t t, int64_t total)
    {
        const std::string f = "adamw.step";
        if (t < 1) raise(PSK_E7001, "adamw.step: steps count from 1");
        for (auto &kv : params) {
            if (!results.count(kv.first)) raise(PSK_E7001, "adamw.step: the gradient has no leaf `" + kv.first + "`");
            if (kv.second.dtype == PSK_I8 || kv.second.scales) raise(PSK_E7005, "adamw.step: `" + kv.first + "` is quantised");
        }
        std::map<std::string, Tensor> grads = results;
        const int shift = adamw.clip ? 14 : 0;
        auto at = [&](int n) { return f + "/%" + std::to_string(n + shift); };
        if (adamw.clip) {
            // %7 sum_squares g (a launch a leaf, the sums added on the host), then [%8 sqrt; %11 + 1e-6; %14 c / it;
            // %17 1 - it; %18 relu; %19 1 - it] as one scalar group, %20 g * factor leaf by leaf
            double acc = 0.0;
            std::vector<Tensor> sums; // every leaf's launch first, then one wait for all of them
            for (auto &kv : params) {
                Tensor n2 = reduce_all(f + "/%7", PSK_REDUCE_SUMSQ, grads[kv.first]);
                Tensor wide = fresh({}, PSK_F64);
                convert_into(n2, wide);
                sums.push_back(wide);
            }
            for (auto &wide : sums) {
                double v = 0.0;
                check(vt->download(vt->self, &v, wide.ptr(), 8), "download");
                acc += v;
            }
            check(vt->sync(vt->self), "sum_squares");
            Tensor n2 = scalar(f + "/%7", acc), tiny = scalar(f + "/%10", 1e-6), c = scalar(f + "/%13", adamw.grad_clip), one1 = scalar(f + "/%16", 1.0);
            Tensor factor = fused(f + "/%19", {U(PSK_SQRT, 0), Bn(PSK_ADD, S(0), 1), Bn(PSK_DIV, 2, S(1)), Bn(PSK_SUB, 3, S(2)), U(PSK_RELU, S(3)), Bn(PSK_SUB, 3, S(4))}, {&n2, &tiny, &c, &one1});
            for (auto &kv : params) grads[kv.first] = binary(f + "/%20", PSK_MUL, grads[kv.first], factor);
        }
        Tensor one = scalar(at(8), 1.0), b1 = scalar(at(10), adamw.beta1), b2 = scalar(at(12), adamw.beta2);
        Tensor omb1 = binary(at(13), PSK_SUB, one, b1), omb2 = binary(at(14), PSK_SUB, one, b2);
        Tensor tr = scalar(at(22), (double)t);
        // 1 - exp(t · ln β)
        auto bias_correction = [&](const std::string &site, const Tensor &beta) {
            return fused(site, {U(PSK_LOG, 0), Bn(PSK_MUL, 1, S(0)), U(PSK_EXP, S(1)), Bn(PSK_SUB, 2, S(2))}, {&beta, &tr, &one});
        };
        Tensor bc1 = bias_correction(at(26), b1), bc2 = bias_correction(at(30), b2);
        Tensor eps = scalar(at(35), adamw.eps), lambda = scalar(at(39), adamw.weight_decay);
        Tensor lr = adamw_lr(t, total);
        std::map<std::string, Tensor> next;
        results.clear();
        for (auto &kv : params) {
            const std::string &path = kv.first;
            Tensor theta = kv.second, g = grads[path];
            g.axes = theta.axes;
            if (!moment_m.count(path)) { // adamw.init: zeros_like θ
                moment_m[path] = zeros(at(17), theta.axes);
                moment_v[path] = zeros(at(21), theta.axes);
            }
            const Tensor &m = moment_m[path], &v = moment_v[path];
            Tensor m2 = fused(at(17), {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 3), Bn(PSK_ADD, S(0), S(1))}, {&m, &b1, &g, &omb1});
            Tensor v2 = fused(at(21), {Bn(PSK_MUL, 0, 1), Bn(PSK_MUL, 2, 2), Bn(PSK_MUL, S(1), 3), Bn(PSK_ADD, S(0), S(2))}, {&v, &b2, &g, &omb2});
            // m̂ = m'/bc1, v̂ = v'/bc2, √v̂, + ε, m̂ / that, θ·λ, their sum, × lr, θ - that
            Tensor theta2 = fused(at(44), {Bn(PSK_DIV, 0, 1), Bn(PSK_DIV, 2, 3), U(PSK_SQRT, S(1)), Bn(PSK_ADD, S(2), 4), Bn(PSK_DIV, S(0), S(3)), Bn(PSK_MUL, 5, 6), Bn(PSK_ADD, S(4), S(5)), Bn(PSK_MUL, S(6), 7), Bn(PSK_SUB, 5, S(7))},
                                  {&m2, &bc1, &v2, &bc2, &eps, &theta, &lambda, &lr});
            if (theta2.dtype != theta.dtype) { // a parameter stays in its own storage type
                Tensor back = fresh(theta.axes, theta.dtype);
                convert_into(theta2, back);
                theta2 = back;
            }
            next[path] = theta2;
            moment_m[path] = m2;
            moment_v[path] = v2;
            results[path] = theta2;
            results["m:" + path] = m2;
            results["v:" + path] = v2;
        }
        for (auto &kv : next) params[kv.first] = kv.second;
    }

    // x·w then a row LayerNorm: %0 θ, %1 x, %2 w; %3 dot; LayerNorm.apply on it.
    Tensor contract_ln(const Tensor &x, const Tensor &w)
    {
        Tensor y = dot("contract_ln/%3", x, w);
        y.axes.back().name = "model";
        return layernorm(param("ln.γ"), param("ln.β"), y, 1e-5);
    }


    // ===========================================================================
    // examples/corpus/nlp/05_gpt.psk (the GPT workload). Outside training a dropout is
    // a mask of ones, made by the host, and the product with it is still a launch
    // (host.rs:1626).
    // ===========================================================================
    std::map<std::string, Tensor> ones_cache;
    Tensor ones_like(const std::string &site, const Tensor &x)
    {
        int d = site_dtype(site);
        std::string key = show(x.axes) + "|" + std::to_string(d);
        auto hit = ones_cache.find(key);
        if (hit != ones_cache.end()) return hit->second;
        Tensor out = fresh(x.axes, d);
        psk_launch l;
        memset(&l, 0, sizeof l);
        l.op = PSK_OP_IOTA;
        l.kind = PSK_IOTA_FILL;
        l.dtype = d;
        l.fparam[0] = 1.0;
        set_space(l, x.axes, {});
        set_operand(l.out, out, contiguous(x.axes), {});
        int64_t before = launches;
        std::string keep = log;
        run(l, "dropout_mask", {}, out);
        launches = before;
        log = keep;
        ones_cache[key] = out;
        return out;
    }

    // 05_gpt.psk LayerNorm: %0 θ, %1 x; μ %2, sub %3, pow %4, σ2 %5, sub %6, lit %7, real %8, add %9, sqrt %10, div %11, γ %12, mul %13, β %14, add %15
    Tensor gpt_layernorm(const Tensor &gamma, const Tensor &beta, const Tensor &x)
    {
        const std::string f = "LayerNorm.apply";
        Tensor mu = reduce_axis(f + "/%2", PSK_REDUCE_MEAN, "model", x);
        Tensor d2 = fused(f + "/%4", {Bn(PSK_SUB, 0, 1), U(PSK_POW, S(0), 2)}, {&x, &mu});
        Tensor var = reduce_axis(f + "/%5", PSK_REDUCE_MEAN, "model", d2);
        Tensor eps = scalar(f + "/%8", 1e-5);
        Tensor sd = fused(f + "/%10", {Bn(PSK_ADD, 0, 1), U(PSK_SQRT, S(0))}, {&var, &eps});
        return fused(f + "/%15", {Bn(PSK_SUB, 0, 1), Bn(PSK_DIV, S(0), 2), Bn(PSK_MUL, S(1), 3), Bn(PSK_ADD, S(2), 4)}, {&x, &mu, &sd, &gamma, &beta});
    }

    Tensor gpt_linear(const std::string &prefix, int64_t l, const Tensor &x)
    {
        Tensor y = dot("Linear.apply/%3", x, layer(param(prefix + ".w"), l));
        return binary("Linear.apply/%5", PSK_ADD, y, layer(param(prefix + ".b"), l));
    }

    // SelfAttention.apply: %0 θ, %1 x, %2 mask, %3 kd
    Tensor gpt_attention(int64_t l, const Tensor &x, const Tensor &mask)
    {
        const std::string f = "SelfAttention.apply";
        const int64_t D = C("D"), H = C("H"), HD = D / H;
        Tensor q = split_heads(f + "/%6", H, HD, gpt_linear("blocks.attn.wq", l, x));
        Tensor k = split_heads(f + "/%9", H, HD, gpt_linear("blocks.attn.wk", l, x));
        Tensor v = split_heads(f + "/%12", H, HD, gpt_linear("blocks.attn.wv", l, x));
        Tensor se = ein(f + "/%13", {"batch", "heads", "seq", "seq2"}, {{"batch", "heads", "seq", "hd"}, {"batch", "heads", "seq2", "hd"}}, {&q, &k});
        Tensor hdr = scalar(f + "/%15", (double)HD);
        Tensor rt = unary(f + "/%16", PSK_SQRT, hdr);
        Tensor s = binary(f + "/%17", PSK_DIV, se, rt);
        Tensor sm = softmax(f + "/%18", "seq2", s, &mask);
        Tensor ones = ones_like(f + "/%20", sm);
        Tensor a = binary(f + "/%21", PSK_MUL, sm, ones);
        Tensor o = ein(f + "/%22", {"batch", "heads", "seq", "hd"}, {{"batch", "heads", "seq", "seq2"}, {"batch", "heads", "seq2", "hd"}}, {&a, &v});
        Tensor m = merge_heads(f + "/%23", H, HD, o);
        return gpt_linear("blocks.attn.wo", l, m);
    }

    // Block.apply: %0 θ, %1 s, %2 mask
    Tensor gpt_block(int64_t l, const Tensor &x, const Tensor &mask)
    {
        const std::string f = "Block.apply";
        Tensor n1 = gpt_layernorm(layer(param("blocks.ln1.γ"), l), layer(param("blocks.ln1.β"), l), x);
        Tensor at = gpt_attention(l, n1, mask);
        Tensor ones = ones_like(f + "/%19", at);
        Tensor h = fused(f + "/%21", {Bn(PSK_MUL, 0, 1), Bn(PSK_ADD, 2, S(0))}, {&at, &ones, &x});
        Tensor n2 = gpt_layernorm(layer(param("blocks.ln2.γ"), l), layer(param("blocks.ln2.β"), l), h);
        Tensor up = gpt_linear("blocks.ff.up", l, n2);
        Tensor g = unary("FeedForward.apply/%4", PSK_GELU, up);
        Tensor dn = gpt_linear("blocks.ff.down", l, g);
        Tensor ones2 = ones_like(f + "/%27", dn);
        return fused(f + "/%29", {Bn(PSK_MUL, 0, 1), Bn(PSK_ADD, 2, S(0))}, {&dn, &ones2, &h});
    }

    // GPT.apply: %0 θ, %1 ids, %2 k
    Tensor gpt_apply(const Tensor &ids)
    {
        const std::string f = "GPT.apply";
        const int64_t T = ids.axes[1].len, L = C("L");
        Tensor mask = causal_mask(f + "/%3", "seq", T);
        Tensor et = embed(f + "/%5", param("tok"), ids);
        Tensor pos = positions(f + "/%7", "seq", T);
        Tensor posw = param("pos");
        if (posw.axes[0].len < T) raise(PSK_E7001, "GPT: the position table has " + std::to_string(posw.axes[0].len) + " rows and the sequence " + std::to_string(T));
        Tensor ep = embed(f + "/%8", posw, pos);
        Tensor ones = ones_like(f + "/%14", et);
        Tensor x = fused(f + "/%15", {Bn(PSK_ADD, 0, 1), Bn(PSK_MUL, S(0), 2)}, {&et, &ep, &ones});
        x.axes.back().name = "model";
        for (int64_t l = 0; l < L; ++l) {
            x = gpt_block(l, x, mask);
            x.axes.back().name = "model";
        }
        Tensor h = gpt_layernorm(param("lnf.γ"), param("lnf.β"), x);
        Tensor logits = dot(f + "/%24", h, param("head"));
        logits.axes.back().name = "vocab";
        return logits;
    }

    Tensor gpt_loss(const Tensor &ids, const Tensor &y)
    {
        Tensor logits = gpt_apply(ids);
        Tensor ce = cross_entropy("loss/%6", logits, y);
        return reduce_all("loss/%7", PSK_REDUCE_MEAN, ce);
    }

    // examples/tests/formats/w8a8.psk: Dense.apply %0 θ, %1 x; a %2 = relu x; w %3; %4 = dot a, w.
    Tensor dense_w8a8(const Tensor &x)
    {
        Tensor a = unary("Dense.apply/%2", PSK_RELU, x);
        return dot("Dense.apply/%4", a, param("w"));
    }

    // values one call computes once where the source computes them again with the same arguments (merged launches)
    std::map<std::pair<void *, int64_t>, std::pair<Tensor, Tensor>> rope_tables;

    Tensor call(const std::string &entry, const std::vector<Tensor> &in)
    {
        struct Forget { psk_host *h; ~Forget() { h->rope_tables.clear(); } } forget{this};
        rope_tables.clear();
        auto need = [&](size_t n) { if (in.size() != n) raise(PSK_E7001, model + "." + entry + " takes " + std::to_string(n) + " inputs"); };
        if (model == "llama") {
            if (entry == "apply") { need(1); return llama_apply(in[0]); }
            if (entry == "loss") { need(2); return llama_loss(in[0], in[1]); }
            if (entry == "loss_grad") { need(2); return llama_loss_grad(in[0], in[1]); }
            if (entry == "prefill") { need(1); return llama_prefill(in[0]); }
            if (entry == "step") { need(1); return llama_step(in[0]); }
            if (entry == "attention" || entry == "attention3") {
                // one attention function on given activations [batch, seq, model], with the causal mask and the
                // angles of its sequence length: examples/spec/rope/rope.psk `attention2` is this with G = H
                need(1);
                // `attention3` (rope.psk:96-97): the base 500 000 and Llama 3's scaling of the frequencies
                const int64_t T = in[0].axes[1].len;
                Tensor mask = causal_mask("Llama.apply/%2", "seq", T);
                const double keep = rope_base;
                if (entry == "attention3") { rope_base = 5e5; rope_llama3 = true; }
                Tensor phi = llama_angles(T);
                rope_base = keep; rope_llama3 = false;
                return llama_attention(0, in[0], mask, phi);
            }
        } else if (model == "gpt") {
            if (entry == "apply") { need(1); return gpt_apply(in[0]); }
            if (entry == "loss") { need(2); return gpt_loss(in[0], in[1]); }
        } else if (model == "mlp") {
            if (entry == "apply") { need(1); return mlp_apply(in[0]); }
            if (entry == "loss") { need(2); return mlp_loss(in[0], in[1]); }
        } else if (model == "layernorm") {
            need(1);
            return layernorm(param("γ"), param("β"), in[0], 1e-5);
        } else if (model == "rmsnorm") {
            need(1);
            return rmsnorm_spec(param("γ"), in[0], 1e-6);
        } else if (model == "toy") {
            if (entry == "loss") { need(1); return toy_loss(in[0]); }
            if (entry == "loss_grad") { need(1); return toy_loss_grad(in[0]); }
        } else if (model == "tower") {
            if (entry == "loss") { need(2); return tower_loss(in[0], in[1]); }
            if (entry == "loss_grad") { need(2); return tower_loss_grad(in[0], in[1]); }
        } else if (model == "mlp_spec") {
            if (entry == "mse") { need(2); return spec_mse(in[0], in[1]); }
            if (entry == "mse_grad") { need(2); return spec_mse_grad(in[0], in[1]); }
        } else if (model == "contract_ln") {
            need(2);
            return contract_ln(in[0], in[1]);
        } else if (model == "dense") {
            need(1);
            return dense_w8a8(in[0]);
        }
        raise(PSK_E7001, "no entry `" + entry + "` of the model `" + model + "`");
    }

    // The axes an entry's input has, by position (the source's types).
    Axes input_axes(const std::string &entry, int i, const psk_value &v)
    {
        std::vector<std::string> names;
        if (model == "llama" && (entry == "attention" || entry == "attention3")) names = {"batch", "seq", "model"};
        else if (model == "llama" || model == "gpt") names = {"batch", "seq"};
        else if (model == "mlp") names = i == 0 ? std::vector<std::string>{"batch", "model"} : std::vector<std::string>{"batch"};
        else if (model == "mlp_spec") names = {"batch", "model"};
        else if (model == "toy") names = {"batch", "seq"};
        else if (model == "tower") names = {"batch", "model"};
        else if (model == "layernorm" || model == "rmsnorm") {
            // ℝ[..., model: D] with a prefix of named axes
            static const char *prefix[] = {"batch", "seq", "a2", "a3", "a4", "a5", "a6"};
            names.assign(v.rank, "");
            for (int k = 0; k + 1 < v.rank; ++k) names[k] = prefix[k];
            if (v.rank) names.back() = "model";
        }
        else if (model == "contract_ln") names = i == 0 ? std::vector<std::string>{"batch", "k"} : std::vector<std::string>{"k", "model"};
        else if (model == "dense") names = {"", ""};
        (void)entry;
        Axes a;
        for (int k = 0; k < v.rank; ++k) a.push_back({k < (int)names.size() ? names[k] : "", v.dims[k]});
        return a;
    }
};

// ===========================================================================
extern "C" {

size_t psk_abi_sizeof(int which)
{
    switch (which) {
    case 0: return sizeof(psk_launch);
    case 1: return sizeof(psk_operand);
    case 2: return sizeof(psk_step);
    case 3: return sizeof(psk_gemm);
    case 4: return sizeof(psk_value);
    case 5: return sizeof(psk_exec_vtable);
    default: return 0;
    }
}

const char *psk_host_error(const psk_host *h) { return h ? h->error.c_str() : g_host_error.c_str(); }

psk_host *psk_host_create(const psk_exec_vtable *exec, const char *realization)
{
    if (!exec || !exec->run) { g_host_error = "no executor"; return nullptr; }
    try {
        psk_host *h = new psk_host;
        h->vt_copy = *exec;
        h->vt = &h->vt_copy;
        h->rz = Realization::parse(realization);
        return h;
    } catch (const HostError &e) {
        g_host_error = "[E" + std::to_string(e.code) + "] " + e.msg; // the code travels in the text: there is no handle to ask
        return nullptr;
    }
}

void psk_host_destroy(psk_host *h) { delete h; }

#define HOST_TRY(h, ...)                       \
    try {                                      \
        __VA_ARGS__;                           \
    } catch (const HostError &e) {             \
        (h)->error = e.msg;                    \
        return e.code;                         \
    }

int psk_host_prepare(psk_host *h, const char *model, const char *consts)
{
    HOST_TRY(h, {
        h->model = model ? model : "";
        static const char *known[] = {"llama", "gpt", "mlp", "mlp_spec", "toy", "tower", "layernorm", "rmsnorm", "contract_ln", "dense"};
        bool ok = false;
        for (auto k : known) ok |= h->model == k;
        if (!ok) raise(PSK_E7001, "no model `" + h->model + "`");
        h->consts.clear();
        std::istringstream ss(consts ? consts : "");
        std::string tok;
        while (ss >> tok) {
            size_t eq = tok.find('=');
            if (eq == std::string::npos) raise(PSK_E7001, "a constant is NAME=N, not `" + tok + "`");
            h->consts[tok.substr(0, eq)] = strtoll(tok.c_str() + eq + 1, nullptr, 10);
        }
        // Realization::check_params (presk-rt/src/lib.rs:688-703): a path that names no parameter is refused
        if (h->model == "llama") {
            static const char *paths[] = {"tok", "head", "norm.γ", "blocks.n1.γ", "blocks.n2.γ", "blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w"};
            for (auto *m : {&h->rz.params})
                for (auto &kv : *m) {
                    bool found = false;
                    for (auto p : paths) found |= kv.first == p;
                    if (!found) raise(PSK_E7001, "the realization's `params` names `" + kv.first + "`, which is no parameter of Llama");
                }
            for (auto &kv : h->rz.quant) {
                bool found = false;
                for (auto p : paths) found |= kv.first == p;
                if (!found) raise(PSK_E7001, "the realization's `quant` names `" + kv.first + "`, which is no parameter of Llama");
            }
        }
    });
    return PSK_OK;
}

int psk_host_set_param(psk_host *h, const char *path, const void *host, int32_t host_dtype, const int64_t *dims, int32_t rank)
{
    HOST_TRY(h, {
        if (host_dtype != PSK_F32 && host_dtype != PSK_F64) raise(PSK_E7001, "a parameter is given as f32 or f64 reals");
        Axes axes;
        for (int i = 0; i < rank; ++i) axes.push_back({"", dims[i]});
        Tensor raw = h->fresh(axes, host_dtype);
        h->check(h->vt->upload(h->vt->self, raw.ptr(), host, (size_t)raw.numel() * elem_bytes(host_dtype)), "upload");
        h->store_param(path, raw);
    });
    return PSK_OK;
}

int psk_host_init_param(psk_host *h, const char *path, uint64_t seed, double std, const int64_t *dims, int32_t rank)
{
    HOST_TRY(h, {
        if (!h->vt->init_normal) raise(PSK_E7005, "this executor draws no parameters");
        Axes axes;
        for (int i = 0; i < rank; ++i) axes.push_back({"", dims[i]});
        bool quant;
        QuantSpec qs;
        int d = h->param_dtype(path, quant, qs);
        // drawn as f32, then stored as the realization says; a type narrower than f32 that is not
        // quantised is drawn directly, which rounds the same f32 once
        Tensor raw = h->fresh(axes, quant ? PSK_F32 : d);
        h->check(h->vt->init_normal(h->vt->self, raw.ptr(), raw.dtype, raw.numel(), seed, std), "init");
        h->store_param(path, raw);
    });
    return PSK_OK;
}

static Tensor upload_value(psk_host *h, const char *entry, int i, const psk_value &v)
{
    bool is_index = v.dtype == PSK_I64;
    Axes axes = h->input_axes(entry, i, v);
    Tensor t = h->fresh(axes, v.dtype, is_index, 0);
    h->check(h->vt->upload(h->vt->self, t.ptr(), v.data, (size_t)t.numel() * elem_bytes(t.dtype)), "upload");
    if (is_index || v.dtype == h->rz.dflt) return t;
    // Backend::call realizes every real leaf at the default type (host.rs:654-666)
    Tensor r = h->fresh(axes, h->rz.dflt);
    h->convert_into(t, r);
    return r;
}

int psk_host_call(psk_host *h, const char *entry, const psk_value *inputs, int32_t n_inputs, void *out_host, int32_t out_dtype, int64_t out_capacity, int64_t *out_numel)
{
    HOST_TRY(h, {
        h->launches = 0;
        h->log.clear();
        std::vector<Tensor> in;
        for (int i = 0; i < n_inputs; ++i) in.push_back(upload_value(h, entry, i, inputs[i]));
        Tensor r = h->call(entry, in);
        if (out_numel) *out_numel = r.numel();
        if (r.numel() > out_capacity) raise(PSK_E7001, "the result has " + std::to_string(r.numel()) + " elements and the buffer holds " + std::to_string(out_capacity));
        if (r.is_index) {
            h->check(h->vt->download(h->vt->self, out_host, (uint8_t *)r.ptr() + r.off * 8, (size_t)r.numel() * 8), "download");
        } else {
            if (out_dtype != PSK_F32 && out_dtype != PSK_F64) raise(PSK_E7001, "a result is read as f32 or f64");
            Tensor o = r;
            if (r.dtype != out_dtype || r.off != 0 || r.affine) {
                o = h->fresh(r.axes, out_dtype);
                h->convert_into(r, o);
            }
            h->check(h->vt->download(h->vt->self, out_host, o.ptr(), (size_t)o.numel() * elem_bytes(out_dtype)), "download");
        }
        h->check(h->vt->sync(h->vt->self), entry);
        h->last_result = Tensor();
    });
    return PSK_OK;
}

// Backend::call with inputs already on the executor: `inputs[i].data` is a
// device pointer of this host's executor. The result stays on the executor
// until the next call; `*out` points at it.
int psk_host_call_device(psk_host *h, const char *entry, const psk_value *inputs, int32_t n_inputs, void **out, int32_t *out_dtype, int64_t *out_numel)
{
    HOST_TRY(h, {
        h->launches = 0;
        h->log.clear();
        std::vector<Tensor> in;
        for (int i = 0; i < n_inputs; ++i) {
            Tensor t;
            t.axes = h->input_axes(entry, i, inputs[i]);
            t.dtype = inputs[i].dtype;
            t.is_index = inputs[i].dtype == PSK_I64;
            t.raw = const_cast<void *>(inputs[i].data);
            t.borrowed = true;
            if (!t.is_index && t.dtype != h->rz.dflt) {
                Tensor r = h->fresh(t.axes, h->rz.dflt);
                h->convert_into(t, r);
                t = r;
            }
            in.push_back(t);
        }
        h->last_result = h->call(entry, in);
        if (out) *out = (uint8_t *)h->last_result.ptr() + h->last_result.off * (int64_t)elem_bytes(h->last_result.dtype);
        if (out_dtype) *out_dtype = h->last_result.dtype;
        if (out_numel) *out_numel = h->last_result.numel();
    });
    return PSK_OK;
}

// A leaf of the last call's result when that is a tree (a gradient: one leaf a parameter, by the parameter's
// path), read as f32 or f64 reals.
int psk_host_result(psk_host *h, const char *path, void *out_host, int32_t out_dtype, int64_t out_capacity, int64_t *out_numel)
{
    HOST_TRY(h, {
        auto it = h->results.find(path ? path : "");
        if (it == h->results.end()) raise(PSK_E7001, std::string("the last call left no result `") + (path ? path : "") + "`");
        const Tensor &r = it->second;
        if (out_numel) *out_numel = r.numel();
        if (r.numel() > out_capacity) raise(PSK_E7001, "the result has " + std::to_string(r.numel()) + " elements and the buffer holds " + std::to_string(out_capacity));
        if (out_dtype != PSK_F32 && out_dtype != PSK_F64) raise(PSK_E7001, "a result is read as f32 or f64");
        Tensor o = r;
        if (r.dtype != out_dtype || r.off != 0 || r.affine) {
            o = h->fresh(r.axes, out_dtype);
            h->convert_into(r, o);
        }
        h->check(h->vt->download(h->vt->self, out_host, o.ptr(), (size_t)o.numel() * elem_bytes(out_dtype)), "download");
        h->check(h->vt->sync(h->vt->self), "result");
    });
    return PSK_OK;
}

int psk_host_set_result(psk_host *h, const char *path, const void *data, int32_t dtype, const int64_t *dims, int32_t rank)
{
    HOST_TRY(h, {
        if (!path || !data || (dtype != PSK_F32 && dtype != PSK_F64) || rank < 0 || rank > PSK_MAX_RANK) raise(PSK_E7001, "psk_host_set_result: a path and f32 or f64 reals");
        auto p = h->params.find(path);
        if (p == h->params.end()) raise(PSK_E7001, std::string("no parameter `") + path + "`");
        Axes axes;
        for (int i = 0; i < rank; ++i) axes.push_back({"", dims[i]});
        Tensor raw = h->fresh(axes, dtype);
        if (raw.numel() != p->second.numel()) raise(PSK_E7001, std::string("the leaf `") + path + "` has " + std::to_string(p->second.numel()) + " elements");
        h->check(h->vt->upload(h->vt->self, raw.ptr(), data, (size_t)raw.numel() * elem_bytes(dtype)), "upload");
        Tensor leaf = raw;
        if (dtype != h->rz.dflt) {
            leaf = h->fresh(axes, h->rz.dflt);
            h->convert_into(raw, leaf);
        }
        h->results[path] = leaf;
    });
    return PSK_OK;
}

int psk_host_adamw(psk_host *h, const char *hyperparameters)
{
    HOST_TRY(h, { h->adamw_configure(hyperparameters ? hyperparameters : ""); });
    return PSK_OK;
}

int psk_host_adamw_step(psk_host *h, int64_t t, int64_t total)
{
    HOST_TRY(h, {
        h->launches = 0;
        h->log.clear();
        h->adamw_step(t, total);
        h->check(h->vt->sync(h->vt->self), "adamw.step");
    });
    return PSK_OK;
}

int psk_host_adamw_lr(psk_host *h, int64_t t, int64_t total, double *out)
{
    HOST_TRY(h, {
        Tensor lr = h->adamw_lr(t, total);
        Tensor o = h->fresh({}, PSK_F64);
        h->convert_into(lr, o);
        h->check(h->vt->download(h->vt->self, out, o.ptr(), 8), "download");
        h->check(h->vt->sync(h->vt->self), "adamw.lr");
    });
    return PSK_OK;
}

int psk_host_mean_over_ranks(psk_host *h, psk_comm *c, const void *device_scalar, int32_t dtype, double *out)
{
    HOST_TRY(h, {
        if (!c || !device_scalar || !out) raise(PSK_E7001, "psk_host_mean_over_ranks: a communicator, a scalar and somewhere to put the mean");
        // the scalar as a double on the host, summed over the ranks as doubles, divided by their number
        uint8_t raw[8] = {0};
        h->check(h->vt->download(h->vt->self, raw, device_scalar, elem_bytes(dtype)), "download");
        double x;
        switch (dtype) {
        case PSK_F64: memcpy(&x, raw, 8); break;
        case PSK_F32: { float f; memcpy(&f, raw, 4); x = f; break; }
        case PSK_BF16: { uint32_t w = (uint32_t)(raw[0] | (raw[1] << 8)) << 16; float f; memcpy(&f, &w, 4); x = f; break; }
        default: raise(PSK_E7001, "psk_host_mean_over_ranks: a loss is f64, f32 or bf16");
        }
        Storage tmp(h->vt, 8);
        h->check(h->vt->upload(h->vt->self, tmp.p, &x, 8), "upload");
        if (psk_comm_allreduce(c, tmp.p, 1, PSK_F64, PSK_COMM_SUM) != PSK_OK) raise(PSK_E10001, std::string("all-reduce: ") + psk_comm_error(c));
        h->check(h->vt->download(h->vt->self, &x, tmp.p, 8), "download");
        *out = x / (double)psk_comm_size(c);
    });
    return PSK_OK;
}

int psk_host_envelope_allreduce(psk_host *h, psk_comm *c)
{
    HOST_TRY(h, {
        if (!c) raise(PSK_E7001, "psk_host_envelope_allreduce: a communicator");
        if (!h->slots || h->slot_of.empty()) return PSK_OK;
        // words 0 and 3 of a site merge by maximum, words 1 and 2 by minimum: complemented, one maximum does all four
        std::vector<uint32_t> words(h->slot_of.size() * 4);
        h->check(h->vt->sync(h->vt->self), "calibrate");
        h->check(h->vt->download(h->vt->self, words.data(), h->slots->p, words.size() * 4), "calibrate");
        for (size_t i = 0; i < words.size(); i += 4) { words[i + 1] = ~words[i + 1]; words[i + 2] = ~words[i + 2]; }
        h->check(h->vt->upload(h->vt->self, h->slots->p, words.data(), words.size() * 4), "calibrate");
        if (psk_comm_allreduce(c, h->slots->p, (int64_t)words.size(), PSK_COMM_U32, PSK_COMM_MAX) != PSK_OK) raise(PSK_E10001, std::string("all-reduce: ") + psk_comm_error(c));
        h->check(h->vt->download(h->vt->self, words.data(), h->slots->p, words.size() * 4), "calibrate");
        for (size_t i = 0; i < words.size(); i += 4) { words[i + 1] = ~words[i + 1]; words[i + 2] = ~words[i + 2]; }
        h->check(h->vt->upload(h->vt->self, h->slots->p, words.data(), words.size() * 4), "calibrate");
    });
    return PSK_OK;
}

int psk_host_grads_allreduce(psk_host *h, psk_comm *c)
{
    HOST_TRY(h, {
        if (!c) raise(PSK_E7001, "psk_host_grads_allreduce: a communicator");
        const int n = psk_comm_size(c);
        for (auto &kv : h->results) {
            Tensor leaf = kv.second;
            if (leaf.dtype != PSK_F32 && leaf.dtype != PSK_BF16 && leaf.dtype != PSK_F16 && leaf.dtype != PSK_F64) raise(PSK_E7005, "psk_host_grads_allreduce: the leaf `" + kv.first + "` is not stored as a float NCCL sums");
            if (!leaf.vstrides.empty() || leaf.affine) {
                // a view: summed through a contiguous copy
                Tensor flat = h->fresh(leaf.axes, leaf.dtype);
                h->convert_into(leaf, flat);
                leaf = flat;
            }
            void *p = (uint8_t *)leaf.ptr() + leaf.off * (int64_t)elem_bytes(leaf.dtype);
            if (psk_comm_allreduce(c, p, leaf.numel(), leaf.dtype, PSK_COMM_SUM) != PSK_OK) raise(PSK_E10001, std::string("all-reduce of `") + kv.first + "`: " + psk_comm_error(c));
            // every rank's loss is the mean over its own rows (as many on every rank): the whole batch's gradient is the ranks' mean
            kv.second = n > 1 ? h->fused("grads_allreduce/mean", {U(PSK_DIV_N, 0, n)}, {&leaf}) : leaf;
        }
        h->check(h->vt->sync(h->vt->self), "grads_allreduce");
    });
    return PSK_OK;
}

void psk_host_set_calibrating(psk_host *h, int on)
{
    h->calibrating = on != 0;
    if (on) { h->slot_of.clear(); h->slots.reset(); }
}

const char *psk_host_envelope(psk_host *h)
{
    h->envelope_text.clear();
    try {
        if (!h->slots || h->slot_of.empty()) return "";
        std::vector<uint32_t> words(h->slot_of.size() * 4);
        h->check(h->vt->sync(h->vt->self), "calibrate");
        h->check(h->vt->download(h->vt->self, words.data(), h->slots->p, words.size() * 4), "calibrate");
        auto unorder = [](uint32_t u) { uint32_t b = (u >> 31) ? (u ^ 0x80000000u) : ~u; float x; memcpy(&x, &b, 4); return x; };
        auto asf = [](uint32_t b) { float x; memcpy(&x, &b, 4); return x; };
        for (auto &kv : h->slot_of) { // std::map: sorted by site
            const uint32_t *w = &words[(size_t)kv.second * 4];
            char line[256];
            snprintf(line, sizeof line, "%s\t%.9g\t%.9g\t%.9g\t%.9g\n", kv.first.c_str(), asf(w[0]), asf(w[1]), unorder(w[2]), unorder(w[3]));
            h->envelope_text += line;
        }
    } catch (const HostError &e) {
        h->error = e.msg;
        return "";
    }
    return h->envelope_text.c_str();
}

int64_t psk_host_launches(const psk_host *h) { return h->launches; }
const char *psk_host_launch_log(const psk_host *h) { return h->log.c_str(); }
void psk_host_set_logging(psk_host *h, int on) { h->logging = on != 0; }

} // extern "C"
