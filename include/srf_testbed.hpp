// srf_testbed.hpp -- the host side of the render path in C++: the reference's Testbed as its Python module
// exposes it (internal/python_api.cu:84-133, internal/testbed.h:73-117, internal/testbed.cu:42-80,151-171),
// on top of the C-ABI of libsrf_b200.so (srf_abi.h).  Header-only; link with libsrf_b200.so.
//
//   srf_host::Json       a JSON document: parsed from text (comments allowed, as the reference parses its configs)
//                        or from msgpack (the snapshot format, json::from_msgpack in the reference)
//   srf_host::parse_config()  the reference's configuration keys, defaults and error messages -> srf_config_t
//   srf_host::Testbed    load_model_config / load_snapshot / set_nerf_camera_matrix / fov / fov_xy / render and
//                        the public members the reference's drivers set (experiment/*/python/run.py:128-250)
//
// Errors are std::runtime_error with the reference's texts where it has one.  The training half of the
// reference's Testbed (train, load_training_data, save_snapshot) is outside this library: those members throw.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "srf_abi.h"

namespace srf_host {

// ---- JSON value ---------------------------------------------------------------------------------------
class Json {
public:
    enum Type { Null, Bool, Int, Float, String, Binary, Array, Object };

    Json() = default;
    static Json boolean(bool b) { Json j; j.m_type = Bool; j.m_int = b ? 1 : 0; return j; }
    static Json integer(int64_t v) { Json j; j.m_type = Int; j.m_int = v; j.m_float = (double)v; return j; }
    static Json number(double v) { Json j; j.m_type = Float; j.m_float = v; j.m_int = (int64_t)v; return j; }
    static Json string(std::string s) { Json j; j.m_type = String; j.m_str = std::move(s); return j; }
    static Json binary(std::string bytes) { Json j; j.m_type = Binary; j.m_str = std::move(bytes); return j; }
    static Json array() { Json j; j.m_type = Array; return j; }
    static Json object() { Json j; j.m_type = Object; return j; }

    Type type() const { return m_type; }
    bool is_null() const { return m_type == Null; }
    bool is_object() const { return m_type == Object; }
    bool is_array() const { return m_type == Array; }
    bool is_number() const { return m_type == Int || m_type == Float; }
    bool is_string() const { return m_type == String; }
    bool is_binary() const { return m_type == Binary; }

    // object access
    bool contains(const std::string& key) const { return find(key) != nullptr; }
    const Json* find(const std::string& key) const {
        if (m_type != Object) return nullptr;
        for (const auto& kv : m_members) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    // a missing section is an error (the reference would fail on the null it gets from operator[])
    const Json& at(const std::string& key) const {
        const Json* j = find(key);
        if (!j) throw std::runtime_error("configuration: key '" + key + "' not found");
        return *j;
    }
    Json& set(const std::string& key, Json value) {
        if (m_type == Null) m_type = Object;
        for (auto& kv : m_members) if (kv.first == key) { kv.second = std::move(value); return kv.second; }
        m_members.emplace_back(key, std::move(value));
        return m_members.back().second;
    }
    void erase(const std::string& key) {
        for (size_t i = 0; i < m_members.size(); ++i) if (m_members[i].first == key) { m_members.erase(m_members.begin() + i); return; }
    }
    const std::vector<std::pair<std::string, Json>>& members() const { return m_members; }

    // array access
    size_t size() const { return m_type == Array ? m_items.size() : m_type == Object ? m_members.size() : 0; }
    const Json& at(size_t i) const { return m_items.at(i); }
    void push_back(Json v) { if (m_type == Null) m_type = Array; m_items.push_back(std::move(v)); }

    // config.value(key, default) of nlohmann: the member converted to the default's type, or the default
    double value(const std::string& key, double dflt) const { const Json* j = find(key); return j && j->is_number() ? j->as_double() : dflt; }
    float value(const std::string& key, float dflt) const { return (float)value(key, (double)dflt); }
    int64_t value(const std::string& key, int64_t dflt) const { const Json* j = find(key); return j && j->is_number() ? j->as_int() : dflt; }
    int value(const std::string& key, int dflt) const { return (int)value(key, (int64_t)dflt); }
    uint32_t value(const std::string& key, uint32_t dflt) const { return (uint32_t)value(key, (int64_t)dflt); }
    bool value(const std::string& key, bool dflt) const { const Json* j = find(key); return j && j->m_type == Bool ? j->m_int != 0 : dflt; }
    std::string value(const std::string& key, const char* dflt) const { const Json* j = find(key); return j && j->is_string() ? j->m_str : std::string(dflt); }

    double as_double() const { return m_type == Int ? (double)m_int : m_float; }
    int64_t as_int() const { return m_type == Float ? (int64_t)m_float : m_int; }
    bool as_bool() const { return m_int != 0; }
    const std::string& as_string() const { return m_str; }       // also the bytes of a Binary

private:
    Type m_type = Null;
    int64_t m_int = 0;
    double m_float = 0.0;
    std::string m_str;
    std::vector<Json> m_items;
    std::vector<std::pair<std::string, Json>> m_members;
};

// ---- JSON text ------------------------------------------------------------------------------------------
// RFC 8259 plus // and /* */ comments, which the reference enables (json::parse(f, nullptr, true, true)).
class JsonTextParser {
public:
    explicit JsonTextParser(const std::string& text) : s(text) {}
    Json parse() {
        Json v = value();
        skip();
        if (p != s.size()) fail("trailing characters");
        return v;
    }

private:
    const std::string& s;
    size_t p = 0;

    [[noreturn]] void fail(const char* what) const {
        throw std::runtime_error("JSON parse error at offset " + std::to_string(p) + ": " + what);
    }
    void skip() {
        for (;;) {
            while (p < s.size() && (s[p] == ' ' || s[p] == '\t' || s[p] == '\n' || s[p] == '\r')) ++p;
            if (p + 1 < s.size() && s[p] == '/' && s[p + 1] == '/') { while (p < s.size() && s[p] != '\n') ++p; continue; }
            if (p + 1 < s.size() && s[p] == '/' && s[p + 1] == '*') {
                const size_t e = s.find("*/", p + 2);
                if (e == std::string::npos) fail("unterminated comment");
                p = e + 2;
                continue;
            }
            return;
        }
    }
    bool match(const char* word) {
        const size_t n = strlen(word);
        if (s.compare(p, n, word) == 0) { p += n; return true; }
        return false;
    }
    Json value() {
        skip();
        if (p >= s.size()) fail("unexpected end");
        const char c = s[p];
        if (c == '{') return object();
        if (c == '[') return array();
        if (c == '"') return Json::string(string());
        if (match("true")) return Json::boolean(true);
        if (match("false")) return Json::boolean(false);
        if (match("null")) return Json();
        return number();
    }
    Json object() {
        Json o = Json::object();
        ++p;
        skip();
        if (p < s.size() && s[p] == '}') { ++p; return o; }
        for (;;) {
            skip();
            if (p >= s.size() || s[p] != '"') fail("expected a member name");
            std::string key = string();
            skip();
            if (p >= s.size() || s[p] != ':') fail("expected ':'");
            ++p;
            o.set(key, value());
            skip();
            if (p < s.size() && s[p] == ',') { ++p; continue; }
            if (p < s.size() && s[p] == '}') { ++p; return o; }
            fail("expected ',' or '}'");
        }
    }
    Json array() {
        Json a = Json::array();
        ++p;
        skip();
        if (p < s.size() && s[p] == ']') { ++p; return a; }
        for (;;) {
            a.push_back(value());
            skip();
            if (p < s.size() && s[p] == ',') { ++p; continue; }
            if (p < s.size() && s[p] == ']') { ++p; return a; }
            fail("expected ',' or ']'");
        }
    }
    static void append_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
        else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    }
    uint32_t hex4() {
        if (p + 4 > s.size()) fail("bad \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = s[p++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        std::string out;
        ++p;
        while (p < s.size() && s[p] != '"') {
            char c = s[p++];
            if (c != '\\') { out += c; continue; }
            if (p >= s.size()) fail("bad escape");
            c = s[p++];
            switch (c) {
            case '"': out += '"'; break; case '\\': out += '\\'; break; case '/': out += '/'; break;
            case 'b': out += '\b'; break; case 'f': out += '\f'; break; case 'n': out += '\n'; break;
            case 'r': out += '\r'; break; case 't': out += '\t'; break;
            case 'u': {
                uint32_t cp = hex4();
                if (cp >= 0xD800 && cp < 0xDC00 && p + 1 < s.size() && s[p] == '\\' && s[p + 1] == 'u') {
                    p += 2;
                    cp = 0x10000 + ((cp - 0xD800) << 10) + (hex4() - 0xDC00);
                }
                append_utf8(out, cp);
            } break;
            default: fail("bad escape");
            }
        }
        if (p >= s.size()) fail("unterminated string");
        ++p;
        return out;
    }
    Json number() {
        const size_t start = p;
        bool is_float = false;
        if (p < s.size() && (s[p] == '-' || s[p] == '+')) ++p;
        while (p < s.size() && ((s[p] >= '0' && s[p] <= '9') || s[p] == '.' || s[p] == 'e' || s[p] == 'E' || s[p] == '-' || s[p] == '+')) {
            if (s[p] == '.' || s[p] == 'e' || s[p] == 'E') is_float = true;
            ++p;
        }
        if (p == start) fail("unexpected character");
        const std::string tok = s.substr(start, p - start);
        try {
            if (!is_float) return Json::integer(std::stoll(tok));
            return Json::number(std::stod(tok));
        } catch (const std::exception&) {
            fail("bad number");
        }
    }
};

// ---- msgpack ----------------------------------------------------------------------------------------------
// The subset a JSON document maps to (nil, bool, ints, float32/64, str, bin, array, map with string keys), which
// is what json::to_msgpack writes and json::from_msgpack reads.
class MsgpackReader {
public:
    MsgpackReader(const unsigned char* data, size_t n) : d(data), n(n) {}
    Json parse() { Json v = value(); return v; }

private:
    const unsigned char* d;
    size_t n, p = 0;

    [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("msgpack parse error: ") + what); }
    void need(size_t k) const { if (p + k > n) fail("truncated input"); }
    uint64_t be(int bytes) {
        need((size_t)bytes);
        uint64_t v = 0;
        for (int i = 0; i < bytes; ++i) v = (v << 8) | d[p++];
        return v;
    }
    std::string bytes(size_t k) { need(k); std::string s((const char*)d + p, k); p += k; return s; }
    Json arr(size_t k) { Json a = Json::array(); for (size_t i = 0; i < k; ++i) a.push_back(value()); return a; }
    Json map(size_t k) {
        Json o = Json::object();
        for (size_t i = 0; i < k; ++i) {
            Json key = value();
            if (!key.is_string()) fail("map key is not a string");
            o.set(key.as_string(), value());
        }
        return o;
    }
    Json value() {
        need(1);
        const unsigned char c = d[p++];
        if (c <= 0x7f) return Json::integer(c);
        if (c >= 0xe0) return Json::integer((int8_t)c);
        if (c >= 0x80 && c <= 0x8f) return map(c & 0x0f);
        if (c >= 0x90 && c <= 0x9f) return arr(c & 0x0f);
        if (c >= 0xa0 && c <= 0xbf) return Json::string(bytes(c & 0x1f));
        switch (c) {
        case 0xc0: return Json();
        case 0xc2: return Json::boolean(false);
        case 0xc3: return Json::boolean(true);
        case 0xc4: return Json::binary(bytes((size_t)be(1)));
        case 0xc5: return Json::binary(bytes((size_t)be(2)));
        case 0xc6: return Json::binary(bytes((size_t)be(4)));
        case 0xca: { const uint32_t u = (uint32_t)be(4); float f; memcpy(&f, &u, 4); return Json::number((double)f); }
        case 0xcb: { const uint64_t u = be(8); double f; memcpy(&f, &u, 8); return Json::number(f); }
        case 0xcc: return Json::integer((int64_t)be(1));
        case 0xcd: return Json::integer((int64_t)be(2));
        case 0xce: return Json::integer((int64_t)be(4));
        case 0xcf: return Json::integer((int64_t)be(8));
        case 0xd0: return Json::integer((int8_t)be(1));
        case 0xd1: return Json::integer((int16_t)be(2));
        case 0xd2: return Json::integer((int32_t)be(4));
        case 0xd3: return Json::integer((int64_t)be(8));
        case 0xd9: return Json::string(bytes((size_t)be(1)));
        case 0xda: return Json::string(bytes((size_t)be(2)));
        case 0xdb: return Json::string(bytes((size_t)be(4)));
        case 0xdc: return arr((size_t)be(2));
        case 0xdd: return arr((size_t)be(4));
        case 0xde: return map((size_t)be(2));
        case 0xdf: return map((size_t)be(4));
        default: fail("unsupported type byte (extension types do not occur in a JSON document)");
        }
    }
};

inline void msgpack_write(const Json& j, std::string& out) {
    auto be = [&](uint64_t v, int bytes) { for (int i = bytes - 1; i >= 0; --i) out += (char)((v >> (8 * i)) & 0xff); };
    switch (j.type()) {
    case Json::Null: out += (char)0xc0; break;
    case Json::Bool: out += (char)(j.as_bool() ? 0xc3 : 0xc2); break;
    case Json::Int: {
        const int64_t v = j.as_int();
        if (v >= 0 && v <= 0x7f) out += (char)v;
        else if (v < 0 && v >= -32) out += (char)(int8_t)v;
        else if (v >= 0 && v <= 0xffffffffll) { out += (char)0xce; be((uint64_t)v, 4); }
        else { out += (char)0xd3; be((uint64_t)v, 8); }
    } break;
    case Json::Float: { out += (char)0xcb; const double f = j.as_double(); uint64_t u; memcpy(&u, &f, 8); be(u, 8); } break;
    case Json::String: { out += (char)0xdb; be(j.as_string().size(), 4); out += j.as_string(); } break;
    case Json::Binary: { out += (char)0xc6; be(j.as_string().size(), 4); out += j.as_string(); } break;
    case Json::Array: { out += (char)0xdd; be(j.size(), 4); for (size_t i = 0; i < j.size(); ++i) msgpack_write(j.at(i), out); } break;
    case Json::Object: {
        out += (char)0xdf; be(j.size(), 4);
        for (const auto& kv : j.members()) { msgpack_write(Json::string(kv.first), out); msgpack_write(kv.second, out); }
    } break;
    }
}

inline std::string read_file(const std::string& path, bool binary) {
    std::ifstream f(path, binary ? (std::ios::in | std::ios::binary) : std::ios::in);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

inline std::string lower(std::string s) { for (char& c : s) if (c >= 'A' && c <= 'Z') c = (char)(c - 'A' + 'a'); return s; }

// ---- configuration ------------------------------------------------------------------------------------------
// The sections the reference reads (internal/testbed.cu:65-76) with its keys -- "samlper" is its spelling --, its
// defaults (internal/sampler/occupancy_sampler.cu:909-944, internal/render/ray_marcher.cu:294-301,
// internal/network/ngp_network.h:597-637) and its error messages.
inline int warping_type_from_string(const std::string& str) {           // occupancy_sampler.cu:865-881
    const std::string s = lower(str);
    if (s == "ngp") return SRF_WARP_NGP;
    if (s == "mipnerf360") return SRF_WARP_MIPNERF360;
    if (s == "donerf") return SRF_WARP_DONERF;
    if (s == "sigmoid") return SRF_WARP_SIGMOID;
    if (s == "erp") return SRF_WARP_ERP;
    if (s == "sinusoidalprojection") return SRF_WARP_SINUSOIDAL;
    throw std::runtime_error("Unknown warping type.");
}
inline int sampling_type_from_string(const std::string& str) {          // :883-893
    const std::string s = lower(str);
    if (s == "original") return SRF_SAMPLING_ORIGINAL;
    if (s == "disparity") return SRF_SAMPLING_DISPARITY;
    if (s == "log") return SRF_SAMPLING_LOG;
    throw std::runtime_error("Unknown sampling type.");
}
inline int griddist_type_from_string(const std::string& str) {          // :895-907; the constructor's default "Exp" throws too
    const std::string s = lower(str);
    if (s == "warpedspace_exp") return SRF_GRID_WARPED_EXP;
    if (s == "warpedspace_reciprocal") return SRF_GRID_WARPED_RECIPROCAL;
    if (s == "metricspace_exp") return SRF_GRID_METRIC_EXP;
    if (s == "metricspace_reciprocal") return SRF_GRID_METRIC_RECIPROCAL;
    throw std::runtime_error("Unknown grid distribution type.");
}
inline int loss_type_from_string(const std::string& str) {              // internal/utils/loss.cu:100-118
    const std::string s = lower(str);
    if (s == "l2") return SRF_LOSS_L2;
    if (s == "relativel2") return SRF_LOSS_RELATIVE_L2;
    if (s == "l1") return SRF_LOSS_L1;
    if (s == "mape") return SRF_LOSS_MAPE;
    if (s == "smape") return SRF_LOSS_SMAPE;
    if (s == "smoothl1") return SRF_LOSS_SMOOTH_L1;
    if (s == "logl1") return SRF_LOSS_LOG_L1;
    throw std::runtime_error("Unknown loss type.");
}

inline srf_config_t parse_config(const Json& model_config) {
    srf_config_t c;
    srf_config_default(&c);
    const Json& s = model_config.at("samlper");
    c.warping_type = warping_type_from_string(s.value("warping_type", "NGP"));
    c.aabb_scale = s.value("aabb_scale", 1u);
    c.use_grid = s.value("use_grid", true) ? 1 : 0;
    if (c.use_grid) {
        c.grid_size = s.value("grid_size", 128u);
        c.num_cascades = s.value("num_cascades", 1u);
        c.ema_decay = s.value("ema_decay", 0.95f);
        c.grid_distribution_type = griddist_type_from_string(s.value("grid_distribution_type", "Exp"));
    }
    c.maximum_marching_steps = s.value("maximum_marching_steps", 1024u);
    c.cone_angle_constant = s.value("cone_angle_constant", 0.f);
    c.min_cone_stepsize = s.value("min_cone_stepsize", 0.f);         // 0: the library derives the reference's default
    c.max_cone_stepsize = s.value("max_cone_stepsize", 0.f);
    c.near_distance = s.value("near_distance", 0.2f);
    c.far_distance = s.value("far_distance", 100.f);
    c.sampling_type = sampling_type_from_string(s.value("sampling_type", "Original"));
    c.snap_to_pixel_centers_in_rendering = s.value("snap_to_pixel_centers_in_rendering", true) ? 1 : 0;
    c.min_optical_thickness = s.value("min_optical_thickness", 0.01f);
    static const Json empty = Json::object();
    const Json& r = model_config.contains("render") ? model_config.at("render") : empty;
    c.transmittance_threshold = r.value("transmittance_threshold", 0.0001f);
    c.train_in_linear_color = r.value("train_in_linear_color", false) ? 1 : 0;
    const Json& net = model_config.at("network");
    const Json& enc = net.at("encoding");
    const uint32_t fpl = enc.value("n_features_per_level", 2u);
    uint32_t n_levels = enc.value("n_levels", 16u);
    if (enc.contains("n_features") && enc.value("n_features", 0u) > 0) n_levels = enc.value("n_features", 0u) / fpl;
    c.n_levels = n_levels;
    c.n_features_per_level = fpl;
    c.log2_hashmap_size = enc.value("log2_hashmap_size", 15u);
    const uint32_t base = enc.value("base_resolution", 0u);
    c.base_resolution = base ? base : (1u << (c.log2_hashmap_size / 3));
    c.desired_resolution = enc.value("desired_resolution", 2048.0f);
    c.per_level_scale = enc.value("per_level_scale", 0.0f);
    for (const char* key : {"network", "rgb_network"})
        if (net.at(key).value("n_neurons", 64u) != 64u)
            throw std::runtime_error("this library implements the 64-neuron MLPs every shipped config uses");
    if (net.at("network").value("n_hidden_layers", 1u) != 1u || net.at("rgb_network").value("n_hidden_layers", 2u) != 2u)
        throw std::runtime_error("this library implements 1 hidden density layer and 2 hidden colour layers");
    if (net.at("dir_encoding").value("degree", 4u) != 4u)
        throw std::runtime_error("this library implements spherical harmonics of degree 4");
    return c;
}

// ---- snapshots ----------------------------------------------------------------------------------------------
// What Testbed::save_snapshot adds to the configuration document (internal/testbed.cu:135-149):
//   snapshot.scene_scale, snapshot.scene_offset [x,y,z] (internal/utils/json_binding.h:13-26),
//   snapshot.density_grid: cells * cascades fp32 in Morton order, as binary,
//   snapshot.n_params / params_type ("__half" | "float") / params_binary: the trainer's parameter vector in the
//   network's order (internal/network/ngp_network.h:491-536): density MLP, colour MLP, hash grid.
// The trainer is tiny-cuda-nn's; the three field names and the layout (row-major [out][in] matrices layer after layer,
// the last layer padded to 16 outputs; hash-grid levels one after the other) are that library's published format.
struct Snapshot {
    float scene_scale = 1.f;
    float scene_offset[3] = {0.5f, 0.5f, 0.5f};
    std::vector<float> density_grid;
    std::vector<uint16_t> density_mlp, rgb_mlp, hash_table;      // fp16 bit patterns
};

constexpr size_t kDensityMlpParams = 64 * 32 + 16 * 64;
constexpr size_t kRgbMlpParams = 64 * 32 + 64 * 64 + 16 * 64;

inline uint16_t float_to_half_bits(float f) {                     // round to nearest even, as the device conversion does
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0u));
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);      // rounds to infinity
    if (x < 0x33000001u) return (uint16_t)sign;                   // rounds to zero
    if (x < 0x38800000u) {                                        // subnormal half
        const uint32_t shift = 126u - (x >> 23);                  // 14..24
        const uint32_t mant = (x & 0x7fffffu) | 0x800000u;
        uint32_t h = mant >> shift;
        const uint32_t rem = mant & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (h & 1u))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((x - 0x38000000u) >> 13);
    const uint32_t rem = x & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
}

// Binary members arrive as msgpack bin; some JSON libraries write {"bytes": [...]} instead.
inline std::string binary_of(const Json& j) {
    if (j.is_binary()) return j.as_string();
    if (j.is_object() && j.contains("bytes")) {
        const Json& b = j.at("bytes");
        if (b.is_binary()) return b.as_string();
        std::string s;
        for (size_t i = 0; i < b.size(); ++i) s += (char)b.at(i).as_int();
        return s;
    }
    throw std::runtime_error("ERROR in loading snapshot.");
}

inline Snapshot parse_snapshot(const Json& doc) {
    if (!doc.is_object() || !doc.contains("snapshot")) throw std::runtime_error("ERROR in loading snapshot.");
    const Json& s = doc.at("snapshot");
    Snapshot out;
    out.scene_scale = (float)s.at("scene_scale").as_double();
    const Json& off = s.at("scene_offset");
    for (size_t i = 0; i < 3 && i < off.size(); ++i) out.scene_offset[i] = (float)off.at(i).as_double();
    const std::string grid = binary_of(s.at("density_grid"));
    out.density_grid.resize(grid.size() / 4);
    memcpy(out.density_grid.data(), grid.data(), out.density_grid.size() * 4);
    const std::string ptype = s.value("params_type", "__half");
    const std::string raw = binary_of(s.at("params_binary"));
    std::vector<uint16_t> params;
    if (ptype == "float") {
        params.resize(raw.size() / 4);
        for (size_t i = 0; i < params.size(); ++i) { float f; memcpy(&f, raw.data() + 4 * i, 4); params[i] = float_to_half_bits(f); }
    } else if (ptype == "__half") {
        params.resize(raw.size() / 2);
        memcpy(params.data(), raw.data(), params.size() * 2);
    } else {
        throw std::runtime_error("snapshot parameters of type '" + ptype + "' are not supported");
    }
    const size_t n_params = (size_t)s.value("n_params", (int64_t)params.size());
    if (params.size() < n_params || n_params < kDensityMlpParams + kRgbMlpParams)
        throw std::runtime_error("snapshot parameter vector is shorter than n_params");
    out.density_mlp.assign(params.begin(), params.begin() + kDensityMlpParams);
    out.rgb_mlp.assign(params.begin() + kDensityMlpParams, params.begin() + kDensityMlpParams + kRgbMlpParams);
    out.hash_table.assign(params.begin() + kDensityMlpParams + kRgbMlpParams, params.begin() + n_params);
    return out;
}

// ---- Testbed ---------------------------------------------------------------------------------------------------
// Testbed::RenderingBuffer as Python sees it (internal/python_api.cu:123-133)
struct RenderingBuffer {
    int render_mode = SRF_MODE_SHADE;
    int tonemap_curve = SRF_TONEMAP_IDENTITY;
    float exposure = 0.f;
    int fov_axis = 1;
    float relative_focal_length[2] = {1.f, 1.f};
    float principal_point[2] = {0.5f, 0.5f};
    // kept for drivers that set them; the frame loop here has no compaction rounds (see srf_set_wave_schedule)
    uint32_t MIN_STEPS_INBETWEEN_COMPACTION = 1, MAX_STEPS_INBETWEEN_COMPACTION = 8;
    float camera_matrix[12] = {1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0};     // row-major 3x4, internal convention
};

class Testbed {
public:
    explicit Testbed(int device = 0) : m_device(device) {}
    ~Testbed() { if (m_ctx) srf_destroy(m_ctx); }
    Testbed(const Testbed&) = delete;
    Testbed& operator=(const Testbed&) = delete;

    // public members of the reference's Testbed (internal/testbed.h:113-117)
    int m_loss_type = SRF_LOSS_L2;
    int m_density_activation = SRF_ACT_EXPONENTIAL;
    int m_rgb_activation = SRF_ACT_LOGISTIC;
    float m_background_color[4] = {0.f, 0.f, 0.f, 1.f};
    int m_color_space = SRF_COLOR_LINEAR;
    float m_scene_scale = 1.f;
    float m_scene_offset[3] = {0.5f, 0.5f, 0.5f};
    RenderingBuffer m_rendering_buffer;

    // Testbed::load_model_config (internal/testbed.cu:42-80)
    void load_model_config(const std::string& config_path) {
        std::ifstream probe(config_path);
        if (config_path.empty() || !probe.good()) throw std::runtime_error("The model config must exist.");
        probe.close();
        const size_t dot = config_path.find_last_of('.');
        const std::string ext = dot == std::string::npos ? "" : lower(config_path.substr(dot + 1));
        Json doc;
        if (ext == "json") {
            const std::string text = read_file(config_path, false);
            doc = JsonTextParser(text).parse();
        } else if (ext == "msgpack") {
            const std::string bytes = read_file(config_path, true);
            doc = MsgpackReader((const unsigned char*)bytes.data(), bytes.size()).parse();
        } else {
            throw std::runtime_error("The model config must be a .json or .msgpack file.");
        }
        load_model_config_json(std::move(doc));
    }

    void load_model_config_json(Json doc) {
        srf_config_t cfg = parse_config(doc);
        if (doc.contains("loss") && doc.at("loss").is_string()) m_loss_type = loss_type_from_string(doc.at("loss").as_string());
        m_model_config = std::move(doc);
        m_cfg = cfg;
        rebuild_context();
    }

    // Testbed::load_snapshot (internal/testbed.cu:151-171)
    void load_snapshot(const std::string& snapshot_path) {
        load_model_config(snapshot_path);
        const Snapshot snap = parse_snapshot(m_model_config);
        uint32_t offsets[17];
        check(srf_hashgrid_layout(&m_cfg, offsets, nullptr, nullptr));
        const size_t want = (size_t)offsets[m_cfg.n_levels] * m_cfg.n_features_per_level;
        if (snap.hash_table.size() != want)
            throw std::runtime_error("snapshot holds " + std::to_string(snap.hash_table.size()) +
                                     " hash-grid parameters, the configuration needs " + std::to_string(want));
        m_scene_scale = snap.scene_scale;
        for (int i = 0; i < 3; ++i) m_scene_offset[i] = snap.scene_offset[i];
        load_parameters(snap.hash_table.data(), snap.hash_table.size(), snap.density_mlp.data(), snap.rgb_mlp.data(),
                        snap.density_grid.data(), snap.density_grid.size());
    }

    // What load_snapshot restores, from arrays: parameters, density grid, then update_grid_bitfield (:166-170).
    void load_parameters(const uint16_t* hash_table, size_t n_table, const uint16_t* density_mlp, const uint16_t* rgb_mlp,
                         const float* density_grid, size_t n_grid) {
        need_context();
        check(srf_upload_network(m_ctx, hash_table, n_table, density_mlp, kDensityMlpParams, rgb_mlp, kRgbMlpParams));
        check(srf_upload_density_grid(m_ctx, density_grid, n_grid, nullptr));
        check(srf_update_grid_bitfield(m_ctx, nullptr));
    }

    // fov / fov_xy (internal/testbed.h:73-84, internal/utils/common_device.h:105-121): the setters take radians,
    // the getters return degrees, as in the reference
    float fov() const { return focal_length_to_fov(m_rendering_buffer.relative_focal_length[m_rendering_buffer.fov_axis]); }
    void set_fov(float rad) { m_rendering_buffer.relative_focal_length[0] = m_rendering_buffer.relative_focal_length[1] = fov_to_focal_length(rad); }
    void fov_xy(float out[2]) const { for (int i = 0; i < 2; ++i) out[i] = focal_length_to_fov(m_rendering_buffer.relative_focal_length[i]); }
    void set_fov_xy(const float rad[2]) { for (int i = 0; i < 2; ++i) m_rendering_buffer.relative_focal_length[i] = fov_to_focal_length(rad[i]); }

    // set_nerf_camera_matrix (internal/testbed.h:87-89) = spec_opengl_to_opencv (common_device.h:123-141): negate
    // columns 1 and 2, scale and offset the position.  `cam`: row-major 3x4.
    void set_nerf_camera_matrix(const float cam[12]) {
        float* m = m_rendering_buffer.camera_matrix;
        for (int r = 0; r < 3; ++r) {
            m[r * 4 + 0] = cam[r * 4 + 0];
            m[r * 4 + 1] = cam[r * 4 + 1] * -1.0f;
            m[r * 4 + 2] = cam[r * 4 + 2] * -1.0f;
            m[r * 4 + 3] = cam[r * 4 + 3] * m_scene_scale + m_scene_offset[r];
        }
    }

    // Testbed::render (internal/python_api.cu:17-41): spp passes, then the image as height x width x 4 floats.
    void render(int width, int height, int spp, bool to_srgb, float* h_image, srf_frame_stats_t* stats = nullptr) {
        need_context();
        if (m_cfg.density_activation != m_density_activation || m_cfg.rgb_activation != m_rgb_activation)
            throw std::runtime_error("density_activation / rgb_activation must be set before load_model_config: the context is built with them");
        srf_view_t view;
        memset(&view, 0, sizeof(view));
        memcpy(view.camera, m_rendering_buffer.camera_matrix, sizeof(view.camera));
        view.width = (uint32_t)width; view.height = (uint32_t)height;
        for (int i = 0; i < 2; ++i) {
            view.relative_focal_length[i] = m_rendering_buffer.relative_focal_length[i];
            view.principal_point[i] = m_rendering_buffer.principal_point[i];
        }
        view.render_mode = m_rendering_buffer.render_mode;
        view.depth_scale = 1.f / m_scene_scale;                       // testbed.cu:576
        view.shard_rows = 8; view.shard_count = 1; view.shard_rank = 0;
        srf_post_t post;
        memset(&post, 0, sizeof(post));
        post.exposure = m_rendering_buffer.exposure;
        for (int i = 0; i < 4; ++i) post.background_color[i] = m_background_color[i];
        post.color_space = m_color_space;
        post.tonemap_curve = m_rendering_buffer.tonemap_curve;
        post.to_srgb = to_srgb ? 1 : 0;
        check(srf_render(m_ctx, &view, &post, (uint32_t)spp, h_image, stats));
    }

    // Testbed::train_prep_nerf (internal/testbed.cu:203-239): one density-grid refresh
    void train_prep_nerf(uint32_t training_step) { need_context(); check(srf_refresh_grid(m_ctx, training_step, nullptr)); }

    // the training half is not part of this library
    [[noreturn]] void train(uint32_t, uint32_t) { throw std::runtime_error("training is not part of this library"); }
    [[noreturn]] void load_training_data(const std::string&) { throw std::runtime_error("training is not part of this library"); }
    [[noreturn]] void save_snapshot(const std::string&, bool) { throw std::runtime_error("training is not part of this library: nothing to snapshot"); }

    const srf_config_t& config() const { return m_cfg; }
    const Json& model_config() const { return m_model_config; }
    srf_ctx* context() { return m_ctx; }
    bool has_context() const { return m_ctx != nullptr; }

    static float fov_to_focal_length(float rad) { return 0.5f * 1.0f / tanf(0.5f * rad); }                 // common_device.h:105
    static float focal_length_to_fov(float fl) { return (float)(180.f * 0.63661977236758134308 * atanf(1.0f / (fl * 2.f))); }   // :113-116, M_2_PI

private:
    int m_device;
    srf_ctx* m_ctx = nullptr;
    srf_config_t m_cfg{};
    Json m_model_config;

    void check(srf_status st) const {
        if (st != SRF_OK) throw std::runtime_error(std::string("srf: ") + srf_last_error(m_ctx));
    }
    void need_context() const { if (!m_ctx) throw std::runtime_error("load_model_config first"); }
    void rebuild_context() {
        m_cfg.density_activation = m_density_activation;
        m_cfg.rgb_activation = m_rgb_activation;
        m_cfg.field_type = SRF_FIELD_NETWORK;
        if (m_ctx) { srf_destroy(m_ctx); m_ctx = nullptr; }
        const srf_status st = srf_create(&m_cfg, m_device, &m_ctx);
        if (st != SRF_OK) { m_ctx = nullptr; throw std::runtime_error(std::string("srf: ") + srf_last_error(nullptr)); }
    }
};

}  // namespace srf_host
