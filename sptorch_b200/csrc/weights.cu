// weights.cu -- readers of the reference's on-disk weight formats and the loaders that feed them to a device model.
// Host code only (no kernels); everything here works without a GPU except the final upload.
//
//   .sptc binary checkpoint   crates/serialize/src/lib.rs:15-131   [magic "SPTC" u32][version u32 = 1][count u32] then per
//                             parameter [ndim u32][dims u32...][f32 little-endian data]; no names: order = named_parameters
//   JSON state_dict           serialize/src/lib.rs:172-186, 315-328, 446-481   {"schema": "sptorch.state_dict.v1",
//                             "format_version": 1, "entries": [{"name", "shape", "dtype": "F32"|"F16"|"BF16", "data": [...]}]}
//   manifest beside it        serialize/src/lib.rs:340-441, crates/versioning/src/lib.rs:32-66   "<weights>.manifest.json"
//   safetensors               serialize/src/safetensors.rs:25-73, 118-187   [header bytes u64][JSON header][raw tensor bytes],
//                             F32 / F16 / BF16 converted to f32 exactly as f16_to_f32 / bf16_to_f32 there
// The strictness of the reference is kept: wrong magic, version, schema, count, shape, dtype, duplicate or missing names are
// errors, and nothing is uploaded unless every check has passed.
#include "common.h"
#include "../../include/sptorch_b200_ext.h"
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

namespace spt {

// ---------------- a small JSON reader ----------------
struct Json {
    enum Type { Null, Bool, Num, Str, Arr, Obj, NumArr } type = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;     // file order
    std::vector<float> nums;                           // NumArr: an array whose elements are all numbers (the weight data)
    const Json* get(const char* key) const {
        for (auto& kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

class JsonParser {
public:
    JsonParser(const char* p, const char* end) : p_(p), end_(end) {}
    bool parse(Json* out, std::string* err) {
        if (!value(out, 0)) { *err = err_; return false; }
        ws();
        if (p_ != end_) { *err = "trailing characters after the JSON value"; return false; }
        return true;
    }
private:
    const char *p_, *end_;
    std::string err_;
    void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) p_++; }
    bool bad(const char* m) { if (err_.empty()) err_ = m; return false; }
    bool lit(const char* w) { size_t n = strlen(w); if ((size_t)(end_ - p_) < n || memcmp(p_, w, n)) return bad("bad literal"); p_ += n; return true; }
    static void utf8(std::string* s, unsigned cp) {
        if (cp < 0x80) s->push_back((char)cp);
        else if (cp < 0x800) { s->push_back((char)(0xC0 | (cp >> 6))); s->push_back((char)(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) { s->push_back((char)(0xE0 | (cp >> 12))); s->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s->push_back((char)(0x80 | (cp & 0x3F))); }
        else { s->push_back((char)(0xF0 | (cp >> 18))); s->push_back((char)(0x80 | ((cp >> 12) & 0x3F))); s->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s->push_back((char)(0x80 | (cp & 0x3F))); }
    }
    bool hex4(unsigned* v) {
        if (end_ - p_ < 4) return bad("short \\u escape");
        unsigned r = 0;
        for (int i = 0; i < 4; i++) {
            char c = *p_++;
            r <<= 4;
            if (c >= '0' && c <= '9') r |= c - '0'; else if (c >= 'a' && c <= 'f') r |= c - 'a' + 10; else if (c >= 'A' && c <= 'F') r |= c - 'A' + 10;
            else return bad("bad \\u escape");
        }
        *v = r;
        return true;
    }
    bool string(std::string* s) {
        if (p_ >= end_ || *p_ != '"') return bad("expected a string");
        p_++;
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c != '\\') { s->push_back(c); continue; }
            if (p_ >= end_) return bad("unterminated escape");
            char e = *p_++;
            switch (e) {
                case '"': s->push_back('"'); break;   case '\\': s->push_back('\\'); break; case '/': s->push_back('/'); break;
                case 'b': s->push_back('\b'); break;  case 'f': s->push_back('\f'); break;  case 'n': s->push_back('\n'); break;
                case 'r': s->push_back('\r'); break;  case 't': s->push_back('\t'); break;
                case 'u': {
                    unsigned cp;
                    if (!hex4(&cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        unsigned lo;
                        if (!hex4(&lo)) return false;
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(s, cp);
                    break;
                }
                default: return bad("unknown escape");
            }
        }
        if (p_ >= end_) return bad("unterminated string");
        p_++;
        return true;
    }
    bool number(double* d, float* f) {
        // strtof on the decimal text gives the correctly rounded f32 (serde_json prints the shortest round-trip form)
        char buf[64];
        size_t n = 0;
        while (p_ + n < end_ && n < sizeof(buf) - 1 && (strchr("+-.eE", p_[n]) || (p_[n] >= '0' && p_[n] <= '9'))) n++;
        if (n == 0) return bad("expected a number");
        memcpy(buf, p_, n); buf[n] = 0;
        char* e1 = nullptr;
        *d = strtod(buf, &e1);
        if (e1 != buf + n) return bad("malformed number");
        *f = strtof(buf, nullptr);
        p_ += n;
        return true;
    }
    bool value(Json* out, int depth) {
        if (depth > 64) return bad("nesting too deep");
        ws();
        if (p_ >= end_) return bad("unexpected end of input");
        char c = *p_;
        if (c == '{') {
            out->type = Json::Obj; p_++; ws();
            if (p_ < end_ && *p_ == '}') { p_++; return true; }
            for (;;) {
                ws();
                std::string k;
                if (!string(&k)) return false;
                ws();
                if (p_ >= end_ || *p_ != ':') return bad("expected ':'");
                p_++;
                out->obj.emplace_back(std::move(k), Json());
                if (!value(&out->obj.back().second, depth + 1)) return false;
                ws();
                if (p_ < end_ && *p_ == ',') { p_++; continue; }
                if (p_ < end_ && *p_ == '}') { p_++; return true; }
                return bad("expected ',' or '}'");
            }
        }
        if (c == '[') {
            p_++; ws();
            out->type = Json::Arr;
            if (p_ < end_ && *p_ == ']') { p_++; out->type = Json::NumArr; return true; }
            // arrays of numbers (the bulk of a state_dict) go straight into a float vector
            if (*p_ == '-' || (*p_ >= '0' && *p_ <= '9')) {
                out->type = Json::NumArr;
                for (;;) {
                    ws();
                    double d; float f;
                    if (!number(&d, &f)) return false;
                    out->nums.push_back(f);
                    out->arr.emplace_back();                 // kept so that integer arrays (shapes) can be read exactly
                    out->arr.back().type = Json::Num; out->arr.back().num = d;
                    ws();
                    if (p_ < end_ && *p_ == ',') { p_++; continue; }
                    if (p_ < end_ && *p_ == ']') { p_++; break; }
                    return bad("expected ',' or ']' in a number array");
                }
                if (out->nums.size() > 64) { out->arr.clear(); out->arr.shrink_to_fit(); }   // data arrays: keep only the floats
                return true;
            }
            for (;;) {
                out->arr.emplace_back();
                if (!value(&out->arr.back(), depth + 1)) return false;
                ws();
                if (p_ < end_ && *p_ == ',') { p_++; continue; }
                if (p_ < end_ && *p_ == ']') { p_++; return true; }
                return bad("expected ',' or ']'");
            }
        }
        if (c == '"') { out->type = Json::Str; return string(&out->str); }
        if (c == 't') { out->type = Json::Bool; out->b = true; return lit("true"); }
        if (c == 'f') { out->type = Json::Bool; out->b = false; return lit("false"); }
        if (c == 'n') { out->type = Json::Null; return lit("null"); }
        out->type = Json::Num;
        float f;
        return number(&out->num, &f);
    }
};

// ---------------- the three formats ----------------
struct WeightEntry { std::string name; std::vector<size_t> shape; std::string dtype; std::vector<float> data; };
struct WeightFile { int format = 0; std::vector<WeightEntry> entries; std::string path; };

static bool read_file(const char* path, std::vector<uint8_t>* out) {
    FILE* f = fopen(path, "rb");
    if (!f) { fail_host("weights: cannot open '%s': %s", path, strerror(errno)); return false; }
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (n < 0) { fclose(f); fail_host("weights: cannot size '%s'", path); return false; }
    out->resize((size_t)n);
    size_t got = n ? fread(out->data(), 1, (size_t)n, f) : 0;
    fclose(f);
    if (got != (size_t)n) { fail_host("weights: short read of '%s'", path); return false; }
    return true;
}

static uint32_t rd32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
static float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

// f16_to_f32 of serialize/src/safetensors.rs:156-183
static float half_to_f32(uint16_t bits) {
    uint32_t sign = (bits >> 15) & 1, exp = (bits >> 10) & 0x1F, mant = bits & 0x3FF;
    if (exp == 0) {
        if (mant == 0) return bits_f32(sign << 31);
        int e = 0;
        while ((mant & 0x400) == 0) { mant <<= 1; e--; }
        mant &= 0x3FF;
        return bits_f32((sign << 31) | ((uint32_t)(127 - 15 + 1 + e) << 23) | (mant << 13));
    }
    if (exp == 31) return bits_f32((sign << 31) | (0xFFu << 23) | (mant << 13));
    return bits_f32((sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13));
}

static bool shape_of(const Json* j, std::vector<size_t>* shape) {
    if (!j || (j->type != Json::NumArr && j->type != Json::Arr)) return false;
    for (auto& e : j->arr) {
        if (e.type != Json::Num || e.num < 0 || e.num != (double)(size_t)e.num) return false;
        shape->push_back((size_t)e.num);
    }
    return j->arr.size() == j->nums.size() || j->type == Json::Arr;
}
static size_t numel(const std::vector<size_t>& s) { size_t n = 1; for (size_t d : s) n *= d; return n; }

static bool parse_sptc(const std::vector<uint8_t>& b, WeightFile* w) {
    if (b.size() < 12) return !fail_host("checkpoint: file too small");
    if (rd32(&b[0]) != 0x53505443u) return !fail_host("invalid checkpoint magic");
    if (rd32(&b[4]) != 1) return !fail_host("unsupported checkpoint version %u", rd32(&b[4]));
    const uint32_t count = rd32(&b[8]);
    size_t off = 12;
    for (uint32_t i = 0; i < count; i++) {
        if (off + 4 > b.size()) return !fail_host("checkpoint: truncated at param[%u]", i);
        const uint32_t ndim = rd32(&b[off]); off += 4;
        if (ndim > 8 || off + 4ull * ndim > b.size()) return !fail_host("checkpoint: bad rank %u at param[%u]", ndim, i);
        WeightEntry e;
        for (uint32_t k = 0; k < ndim; k++, off += 4) e.shape.push_back(rd32(&b[off]));
        const size_t n = numel(e.shape);
        if (n > (b.size() - off) / 4) return !fail_host("checkpoint: data of param[%u] runs past the end of the file", i);
        e.data.resize(n);
        memcpy(e.data.data(), &b[off], n * 4);           // little-endian host
        off += n * 4;
        e.dtype = "F32";
        w->entries.push_back(std::move(e));
    }
    return true;
}

static bool parse_state_dict(const std::vector<uint8_t>& b, WeightFile* w) {
    Json root; std::string err;
    JsonParser ps((const char*)b.data(), (const char*)b.data() + b.size());
    if (!ps.parse(&root, &err) || root.type != Json::Obj) return !fail_host("state_dict: invalid JSON: %s", err.c_str());
    const Json* schema = root.get("schema"); const Json* ver = root.get("format_version"); const Json* ents = root.get("entries");
    if (!schema || schema->type != Json::Str || !ver || ver->type != Json::Num || !ents) return !fail_host("state_dict: missing schema, format_version or entries");
    if (schema->str != "sptorch.state_dict.v1") return !fail_host("unsupported state_dict schema %s", schema->str.c_str());
    if (ver->num != 1) return !fail_host("unsupported state_dict version %g", ver->num);
    if (ents->type == Json::NumArr && ents->nums.empty()) return true;
    if (ents->type != Json::Arr) return !fail_host("state_dict: entries is not an array");
    for (auto& e : ents->arr) {
        const Json* name = e.get("name"); const Json* dt = e.get("dtype"); const Json* data = e.get("data");
        WeightEntry we;
        if (e.type != Json::Obj || !name || name->type != Json::Str || !dt || dt->type != Json::Str || !data || data->type != Json::NumArr ||
            !shape_of(e.get("shape"), &we.shape))
            return !fail_host("state_dict: malformed entry");
        if (dt->str != "F32" && dt->str != "F16" && dt->str != "BF16") return !fail_host("unsupported dtype '%s'", dt->str.c_str());
        we.name = name->str; we.dtype = dt->str; we.data = data->nums;
        w->entries.push_back(std::move(we));
    }
    return true;
}

static bool parse_safetensors(const std::vector<uint8_t>& b, WeightFile* w) {
    if (b.size() < 8) return !fail_host("safetensors: file too small");
    uint64_t hs = 0;
    for (int i = 7; i >= 0; i--) hs = (hs << 8) | b[i];
    if (hs > b.size() - 8) return !fail_host("safetensors: header size exceeds file");
    Json root; std::string err;
    JsonParser ps((const char*)&b[8], (const char*)&b[8] + hs);
    if (!ps.parse(&root, &err) || root.type != Json::Obj) return !fail_host("safetensors: invalid header JSON: %s", err.c_str());
    const size_t data_start = 8 + (size_t)hs, data_len = b.size() - data_start;
    for (auto& kv : root.obj) {
        if (kv.first == "__metadata__") continue;
        const Json& v = kv.second;
        const Json* dt = v.get("dtype"); const Json* offs = v.get("data_offsets");
        WeightEntry e;
        std::vector<size_t> o;
        if (v.type != Json::Obj || !dt || dt->type != Json::Str || !shape_of(v.get("shape"), &e.shape) || !shape_of(offs, &o) || o.size() != 2)
            return !fail_host("safetensors: bad tensor info for '%s'", kv.first.c_str());
        if (o[0] > o[1] || o[1] > data_len) return !fail_host("safetensors: data offsets of '%s' are outside the file", kv.first.c_str());
        const uint8_t* src = &b[data_start + o[0]];
        const size_t nbytes = o[1] - o[0];
        e.name = kv.first; e.dtype = dt->str;
        if (dt->str == "F32") {
            if (nbytes % 4) return !fail_host("safetensors: F32 data of '%s' not aligned", kv.first.c_str());
            e.data.resize(nbytes / 4);
            memcpy(e.data.data(), src, nbytes);
        } else if (dt->str == "F16" || dt->str == "BF16") {
            if (nbytes % 2) return !fail_host("safetensors: %s data of '%s' not aligned", dt->str.c_str(), kv.first.c_str());
            e.data.resize(nbytes / 2);
            for (size_t i = 0; i < nbytes / 2; i++) {
                const uint16_t bits = (uint16_t)(src[2 * i] | (src[2 * i + 1] << 8));
                e.data[i] = dt->str == "F16" ? half_to_f32(bits) : bits_f32((uint32_t)bits << 16);
            }
        } else return !fail_host("unsupported dtype: %s", dt->str.c_str());
        if (e.data.size() != numel(e.shape)) return !fail_host("safetensors: '%s' holds %zu values for a shape of %zu", kv.first.c_str(), e.data.size(), numel(e.shape));
        w->entries.push_back(std::move(e));
    }
    return true;
}

// CheckpointManifest beside a JSON state_dict (serialize/src/lib.rs:366-441)
static int check_manifest(const std::string& weights_path, const WeightFile& w, size_t model_params) {
    std::vector<uint8_t> b;
    if (!read_file((weights_path + ".manifest.json").c_str(), &b)) return 1;
    Json m; std::string err;
    JsonParser ps((const char*)b.data(), (const char*)b.data() + b.size());
    if (!ps.parse(&m, &err) || m.type != Json::Obj) return fail_host("manifest: invalid JSON: %s", err.c_str());
    auto str = [&](const char* k) -> const std::string* { const Json* j = m.get(k); return j && j->type == Json::Str ? &j->str : nullptr; };
    auto num = [&](const char* k, double* v) { const Json* j = m.get(k); if (!j || j->type != Json::Num) return false; *v = j->num; return true; };
    for (const char* k : {"schema", "model_name", "save_kind", "weights_file", "state_dict_schema", "note"})
        if (!str(k)) return fail_host("manifest: missing field '%s'", k);
    double fv = 0, pc = 0, ts = 0;
    if (!num("format_version", &fv) || !num("parameter_count", &pc) || !num("created_at_ms", &ts)) return fail_host("manifest: missing numeric field");
    if (*str("schema") != "sptorch.checkpoint_manifest.v1") return fail_host("unsupported checkpoint manifest schema %s", str("schema")->c_str());
    if (fv != 1) return fail_host("unsupported checkpoint manifest version %g", fv);
    if (*str("state_dict_schema") != "sptorch.state_dict.v1") return fail_host("manifest state_dict schema %s does not match expected sptorch.state_dict.v1", str("state_dict_schema")->c_str());
    const size_t slash = weights_path.find_last_of('/');
    const std::string base = slash == std::string::npos ? weights_path : weights_path.substr(slash + 1);
    if (*str("weights_file") != base) return fail_host("manifest weights file %s does not match %s", str("weights_file")->c_str(), weights_path.c_str());
    if ((size_t)pc != model_params) return fail_host("manifest parameter count mismatch: manifest has %zu, model has %zu", (size_t)pc, model_params);
    const Json* names = m.get("parameter_names");
    if (!names || (names->type != Json::Arr && !(names->type == Json::NumArr && names->nums.empty()))) return fail_host("manifest: parameter_names is not an array of strings");
    if (names->arr.size() != w.entries.size()) return fail_host("manifest parameter name count mismatch: manifest has %zu, weights have %zu", names->arr.size(), w.entries.size());
    for (size_t i = 0; i < names->arr.size(); i++)
        if (names->arr[i].type != Json::Str || names->arr[i].str != w.entries[i].name) return fail_host("manifest parameter names do not match loaded state_dict");
    return 0;
}

struct ParamInfo { std::string name; std::vector<size_t> shape; };
// named_parameters of the model behind the handle (defined with the model in gpt.cu)
std::vector<ParamInfo> gpt_param_table(void* gpt);

static std::string shape_str(const std::vector<size_t>& s) {
    std::string r = "[";
    for (size_t i = 0; i < s.size(); i++) r += (i ? ", " : "") + std::to_string(s[i]);
    return r + "]";
}

}  // namespace spt

using namespace spt;

extern "C" {

void* sptorch_ext_weights_open(const char* path, int format) {
    if (!path) { fail_host("weights_open: null path"); return nullptr; }
    std::vector<uint8_t> b;
    if (!read_file(path, &b)) return nullptr;
    if (format == SPT_WEIGHTS_AUTO) {
        size_t i = 0;
        while (i < b.size() && (b[i] == ' ' || b[i] == '\n' || b[i] == '\t' || b[i] == '\r')) i++;
        if (b.size() >= 4 && rd32(&b[0]) == 0x53505443u) format = SPT_WEIGHTS_SPTC;
        else if (i < b.size() && b[i] == '{') format = SPT_WEIGHTS_STATE_DICT;
        else format = SPT_WEIGHTS_SAFETENSORS;
    }
    std::unique_ptr<WeightFile> w(new WeightFile());
    w->format = format; w->path = path;
    bool ok = false;
    if (format == SPT_WEIGHTS_SPTC) ok = parse_sptc(b, w.get());
    else if (format == SPT_WEIGHTS_STATE_DICT) ok = parse_state_dict(b, w.get());
    else if (format == SPT_WEIGHTS_SAFETENSORS) ok = parse_safetensors(b, w.get());
    else fail_host("weights_open: unknown format %d", format);
    return ok ? w.release() : nullptr;
}

void sptorch_ext_weights_close(void* h) { delete (WeightFile*)h; }
int sptorch_ext_weights_format(void* h) { return h ? ((WeightFile*)h)->format : 0; }
size_t sptorch_ext_weights_count(void* h) { return h ? ((WeightFile*)h)->entries.size() : 0; }
static const WeightEntry* entry(void* h, size_t i) { return h && i < ((WeightFile*)h)->entries.size() ? &((WeightFile*)h)->entries[i] : nullptr; }
const char* sptorch_ext_weights_name(void* h, size_t i) { auto* e = entry(h, i); return e ? e->name.c_str() : ""; }
const char* sptorch_ext_weights_dtype(void* h, size_t i) { auto* e = entry(h, i); return e ? e->dtype.c_str() : ""; }
size_t sptorch_ext_weights_ndim(void* h, size_t i) { auto* e = entry(h, i); return e ? e->shape.size() : 0; }
size_t sptorch_ext_weights_dim(void* h, size_t i, size_t k) { auto* e = entry(h, i); return e && k < e->shape.size() ? e->shape[k] : 0; }
size_t sptorch_ext_weights_numel(void* h, size_t i) { auto* e = entry(h, i); return e ? e->data.size() : 0; }
const float* sptorch_ext_weights_data(void* h, size_t i) { auto* e = entry(h, i); return e ? e->data.data() : nullptr; }

size_t sptorch_ext_gpt_param_count(void* gpt) { return gpt ? gpt_param_table(gpt).size() : 0; }
int sptorch_ext_gpt_param_info(void* gpt, size_t i, char* name, size_t name_cap, size_t* dims, size_t* ndim) {
    if (!gpt) return fail_host("gpt_param_info: null model");
    auto t = gpt_param_table(gpt);
    if (i >= t.size()) return fail_host("gpt_param_info: index %zu out of %zu", i, t.size());
    if (name && name_cap) snprintf(name, name_cap, "%s", t[i].name.c_str());
    if (ndim) {
        if (dims) for (size_t k = 0; k < t[i].shape.size() && k < *ndim; k++) dims[k] = t[i].shape[k];
        *ndim = t[i].shape.size();
    }
    return 0;
}

// mapping: n_map pairs (model parameter name, name in the file); only read for safetensors, NULL = same names
int sptorch_ext_gpt_load_weights(void* gpt, void* wh, const char* const* mapping, size_t n_map) {
    if (!gpt || !wh) return fail_host("gpt_load_weights: null argument");
    const WeightFile& w = *(WeightFile*)wh;
    const std::vector<ParamInfo> params = gpt_param_table(gpt);
    std::vector<const WeightEntry*> src(params.size(), nullptr);
    if (w.format == SPT_WEIGHTS_SPTC) {
        // load_checkpoint (serialize/src/lib.rs:65-131): by position
        if (w.entries.size() != params.size()) return fail_host("param count mismatch: checkpoint has %zu, model has %zu", w.entries.size(), params.size());
        for (size_t i = 0; i < params.size(); i++) {
            if (w.entries[i].shape != params[i].shape)
                return fail_host("shape mismatch at param[%zu]: checkpoint %s, model %s", i, shape_str(w.entries[i].shape).c_str(), shape_str(params[i].shape).c_str());
            src[i] = &w.entries[i];
        }
    } else if (w.format == SPT_WEIGHTS_STATE_DICT) {
        // load_state_dict (serialize/src/lib.rs:237-313): by name, everything must match
        if (w.entries.size() != params.size()) return fail_host("state_dict parameter count mismatch: state has %zu, model has %zu", w.entries.size(), params.size());
        std::map<std::string, const WeightEntry*> by_name;
        for (auto& e : w.entries)
            if (!by_name.emplace(e.name, &e).second) return fail_host("state_dict contains duplicate parameter '%s'", e.name.c_str());
        for (size_t i = 0; i < params.size(); i++) {
            auto it = by_name.find(params[i].name);
            if (it == by_name.end()) return fail_host("state_dict missing parameter '%s'", params[i].name.c_str());
            const WeightEntry* e = it->second;
            if (e->shape != params[i].shape) return fail_host("shape mismatch for '%s': state %s, model %s", e->name.c_str(), shape_str(e->shape).c_str(), shape_str(params[i].shape).c_str());
            if (e->dtype != "F32") return fail_host("dtype mismatch for '%s': state %s, model F32", e->name.c_str(), e->dtype.c_str());   // the model's parameters are F32 tensors
            if (e->data.size() != numel(params[i].shape)) return fail_host("data length mismatch for '%s': state %zu, model %zu", e->name.c_str(), e->data.size(), numel(params[i].shape));
            src[i] = e;
        }
    } else if (w.format == SPT_WEIGHTS_SAFETENSORS) {
        // SafeTensorsFile::load_into (serialize/src/safetensors.rs:85-116): explicit (parameter, file name) pairs with a shape check;
        // without a mapping every model parameter is looked up under its own name
        std::map<std::string, const WeightEntry*> by_name;
        for (auto& e : w.entries) by_name[e.name] = &e;
        std::map<std::string, std::string> alias;
        for (size_t i = 0; i < n_map; i++) {
            if (!mapping || !mapping[2 * i] || !mapping[2 * i + 1]) return fail_host("gpt_load_weights: null name in the mapping");
            alias[mapping[2 * i]] = mapping[2 * i + 1];
        }
        for (size_t i = 0; i < params.size(); i++) {
            auto a = alias.find(params[i].name);
            if (n_map && a == alias.end()) continue;                      // with a mapping, only the listed parameters are written
            const std::string& fname = a == alias.end() ? params[i].name : a->second;
            auto it = by_name.find(fname);
            if (it == by_name.end()) return fail_host("tensor '%s' not found in safetensors", fname.c_str());
            if (it->second->shape != params[i].shape)
                return fail_host("shape mismatch for '%s': safetensors %s, model %s", fname.c_str(), shape_str(it->second->shape).c_str(), shape_str(params[i].shape).c_str());
            src[i] = it->second;
        }
        for (auto& kv : alias) {
            bool known = false;
            for (auto& p : params) known = known || p.name == kv.first;
            if (!known) return fail_host("gpt_load_weights: '%s' is not a parameter of the model", kv.first.c_str());
        }
    } else return fail_host("gpt_load_weights: unknown format %d", w.format);
    // every check has passed: upload
    for (size_t i = 0; i < params.size(); i++)
        if (src[i] && sptorch_ext_gpt_set_param(gpt, params[i].name.c_str(), src[i]->data.data(), src[i]->data.size())) return 1;
    return 0;
}

// load_state_dict_bundle (serialize/src/lib.rs:366-441): manifest checks, then the strict by-name load
int sptorch_ext_gpt_load_bundle(void* gpt, const char* weights_path) {
    if (!gpt || !weights_path) return fail_host("gpt_load_bundle: null argument");
    void* wh = sptorch_ext_weights_open(weights_path, SPT_WEIGHTS_STATE_DICT);
    if (!wh) return 1;
    int rc = check_manifest(weights_path, *(WeightFile*)wh, gpt_param_table(gpt).size());
    if (!rc) rc = sptorch_ext_gpt_load_weights(gpt, wh, nullptr, 0);
    sptorch_ext_weights_close(wh);
    return rc;
}

}  // extern "C"
