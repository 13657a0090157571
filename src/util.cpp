// Error checks, the JSON reader, the safetensors reader and the device pool of the C++ host.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdlib>
#include <fstream>
#include <sstream>

#include "host.hpp"

namespace vllm {
namespace host {

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw Error(std::string(what) + ": " + cudaGetErrorString(e));
}

void kernel_check(int code, const char* what) {
    if (code == 0) return;
    if (code == 10001) throw Error(std::string(what) + ": the kernel refused its arguments");
    if (code == 10002) throw Error(std::string(what) + ": size not supported by this kernel");
    throw Error(std::string(what) + ": CUDA error " + std::to_string(code) + " (" + cudaGetErrorString((cudaError_t)code) + ")");
}

// ------------------------------------------------------------------------------------------------ JSON
namespace json {
namespace {
struct Reader {
    const std::string& s;
    size_t i = 0;
    [[noreturn]] void fail(const char* why) const { throw Error("JSON: " + std::string(why) + " at offset " + std::to_string(i)); }
    void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
    bool eat(char c) { ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return false; }
    void word(const char* w) { size_t n = std::strlen(w); if (s.compare(i, n, w) != 0) fail("unknown word"); i += n; }
    std::string string() {
        std::string out;
        if (s[i] != '"') fail("string expected");
        for (++i; i < s.size() && s[i] != '"'; ++i) {
            if (s[i] != '\\') { out.push_back(s[i]); continue; }
            if (++i >= s.size()) fail("unfinished escape");
            switch (s[i]) {
                case 'n': out.push_back('\n'); break;
                case 't': out.push_back('\t'); break;
                case 'r': out.push_back('\r'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'u': {                                   // kept as UTF-8; tensor names are ASCII
                    if (i + 4 >= s.size()) fail("unfinished \\u");
                    unsigned cp = (unsigned)std::strtoul(s.substr(i + 1, 4).c_str(), nullptr, 16);
                    i += 4;
                    if (cp < 0x80) out.push_back((char)cp);
                    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
                    else { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
                    break;
                }
                default: out.push_back(s[i]);
            }
        }
        if (i >= s.size()) fail("unfinished string");
        ++i;
        return out;
    }
    Value value() {
        ws();
        if (i >= s.size()) fail("value expected");
        Value v;
        const char c = s[i];
        if (c == '{') {
            v.kind = Value::Object;
            ++i;
            if (eat('}')) return v;
            do {
                ws();
                std::string key = string();
                if (!eat(':')) fail("':' expected");
                v.obj.emplace_back(std::move(key), value());
            } while (eat(','));
            if (!eat('}')) fail("'}' expected");
        } else if (c == '[') {
            v.kind = Value::Array;
            ++i;
            if (eat(']')) return v;
            do v.arr.push_back(value()); while (eat(','));
            if (!eat(']')) fail("']' expected");
        } else if (c == '"') {
            v.kind = Value::String;
            v.str = string();
        } else if (c == 't') { word("true"); v.kind = Value::Bool; v.b = true; }
        else if (c == 'f') { word("false"); v.kind = Value::Bool; }
        else if (c == 'n') { word("null"); }
        else {
            const size_t start = i;
            while (i < s.size() && (std::isdigit((unsigned char)s[i]) || s[i] == '-' || s[i] == '+' || s[i] == '.' || s[i] == 'e' || s[i] == 'E')) ++i;
            if (i == start) fail("value expected");
            const std::string tok = s.substr(start, i - start);
            char* end = nullptr;
            v.num = std::strtod(tok.c_str(), &end);
            if (end == tok.c_str() || *end) fail("bad number");
            v.kind = Value::Number;
            v.integral = tok.find_first_of(".eE") == std::string::npos;
        }
        return v;
    }
};
}  // namespace

const Value* Value::find(const std::string& key) const {
    if (kind != Object) return nullptr;
    for (const auto& kv : obj) if (kv.first == key) return &kv.second;
    return nullptr;
}

Value parse(const std::string& text) {
    Reader r{text};
    Value v = r.value();
    r.ws();
    if (r.i != text.size()) r.fail("text after the value");
    return v;
}

Value parse_file(const std::string& path) {
    std::ifstream f(path);
    if (!f) throw Error("Cannot open config: " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    try {
        return parse(ss.str());
    } catch (const Error& e) {
        throw Error(path + " is not valid JSON: " + e.what());
    }
}
}  // namespace json

// ------------------------------------------------------------------------------------------ safetensors
int64_t TensorInfo::numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
}

SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw Error("Cannot open safetensors: " + path);
    struct stat st {};
    if (fstat(fd, &st) != 0 || st.st_size < 8) { ::close(fd); throw Error(path + ": too short for a safetensors file"); }
    size_ = (size_t)st.st_size;
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (map_ == MAP_FAILED) { map_ = nullptr; throw Error(path + ": cannot map the file"); }
    const uint8_t* bytes = static_cast<const uint8_t*>(map_);
    uint64_t header_len = 0;
    std::memcpy(&header_len, bytes, 8);
    if (header_len > size_ - 8) throw Error(path + ": header length " + std::to_string(header_len) + " exceeds the file");
    json::Value header;
    try {
        header = json::parse(std::string(reinterpret_cast<const char*>(bytes + 8), header_len));
    } catch (const Error& e) {
        throw Error(path + ": header is not valid JSON (" + e.what() + ")");
    }
    if (header.kind != json::Value::Object) throw Error(path + ": header is not a JSON object");
    const size_t data_start = 8 + header_len, data_size = size_ - data_start;
    for (const auto& kv : header.obj) {
        if (kv.first == "__metadata__") continue;
        const json::Value *dt = kv.second.find("dtype"), *sh = kv.second.find("shape"), *off = kv.second.find("data_offsets");
        if (!dt || dt->kind != json::Value::String || !sh || sh->kind != json::Value::Array || !off || off->arr.size() != 2)
            throw Error(path + ": tensor '" + kv.first + "' lacks dtype, shape or data_offsets");
        TensorInfo t;
        t.dtype = dt->str;
        for (const auto& d : sh->arr) t.shape.push_back((int64_t)d.num);
        const size_t elem = t.dtype == "F32" ? 4 : (t.dtype == "BF16" || t.dtype == "F16") ? 2 : 0;
        if (!elem) throw Error(path + ": tensor '" + kv.first + "' has type " + t.dtype + "; F32, BF16 and F16 are read");
        const size_t b = (size_t)off->arr[0].num, e = (size_t)off->arr[1].num;
        if (e < b || e > data_size) throw Error(path + ": tensor '" + kv.first + "' lies outside the file");
        if (e - b != (size_t)t.numel() * elem)
            throw Error(path + ": tensor '" + kv.first + "' holds " + std::to_string(e - b) + " bytes, its shape needs " +
                        std::to_string((size_t)t.numel() * elem));
        t.data = bytes + data_start + b;
        t.nbytes = e - b;
        tensors_.emplace(kv.first, std::move(t));
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, size_);
}

// ------------------------------------------------------------------------------------------------ pool
DevicePool::DevicePool(size_t bytes) : total_(bytes) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess)
        throw Error("the device pool of " + std::to_string(bytes) + " bytes could not be allocated: " + cudaGetErrorString(e));
    base_ = static_cast<uint8_t*>(p);
}

DevicePool::~DevicePool() {
    if (base_) cudaFree(base_);
}

void* DevicePool::alloc(size_t bytes, const char* what) {
    const size_t start = rounded(offset_);
    if (start + bytes > total_)
        throw Error(std::string("the device pool has no room for ") + what + ": " + std::to_string(bytes) + " bytes wanted, " +
                    std::to_string(total_ - std::min(total_, start)) + " of " + std::to_string(total_) + " left");
    offset_ = start + bytes;
    return base_ + start;
}

// ---------------------------------------------------------------------------- SHA-256 (FIPS 180-4), for tensor_key
namespace {
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

// The round constants are the first 32 bits of the fractional parts of the cube roots of the first 64 primes,
// the initial state those of the square roots of the first eight; computed here rather than listed.
struct Sha256Tables {
    uint32_t k[64], h0[8];
    Sha256Tables() {
        int primes[64], n = 0;
        for (int c = 2; n < 64; ++c) {
            bool prime = true;
            for (int d = 2; d * d <= c; ++d) if (c % d == 0) { prime = false; break; }
            if (prime) primes[n++] = c;
        }
        for (int i = 0; i < 64; ++i) k[i] = frac_bits(cbrtl((long double)primes[i]));
        for (int i = 0; i < 8; ++i) h0[i] = frac_bits(sqrtl((long double)primes[i]));
    }
    static uint32_t frac_bits(long double x) {
        x -= floorl(x);
        return (uint32_t)floorl(x * 4294967296.0L);
    }
};

void sha256(const std::string& msg, uint8_t out[32]) {
    static const Sha256Tables t;
    uint32_t h[8];
    std::memcpy(h, t.h0, sizeof h);
    std::string m = msg;
    m.push_back((char)0x80);
    while (m.size() % 64 != 56) m.push_back((char)0);
    const uint64_t bits = (uint64_t)msg.size() * 8;
    for (int i = 7; i >= 0; --i) m.push_back((char)((bits >> (8 * i)) & 0xFF));
    for (size_t off = 0; off < m.size(); off += 64) {
        uint32_t w[64];
        for (int i = 0; i < 16; ++i)
            w[i] = ((uint32_t)(uint8_t)m[off + 4 * i] << 24) | ((uint32_t)(uint8_t)m[off + 4 * i + 1] << 16) |
                   ((uint32_t)(uint8_t)m[off + 4 * i + 2] << 8) | (uint32_t)(uint8_t)m[off + 4 * i + 3];
        for (int i = 16; i < 64; ++i) {
            const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; ++i) {
            const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
            const uint32_t t1 = hh + S1 + ch + t.k[i] + w[i];
            const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), maj = (a & b) ^ (a & c) ^ (b & c);
            const uint32_t t2 = S0 + maj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    for (int i = 0; i < 8; ++i)
        for (int j = 0; j < 4; ++j) out[4 * i + j] = (uint8_t)(h[i] >> (24 - 8 * j));
}
}  // namespace

uint64_t tensor_key(uint64_t seed, const std::string& name) {
    uint8_t digest[32];
    sha256(std::to_string(seed) + ":" + name, digest);
    uint64_t key = 0;
    for (int i = 7; i >= 0; --i) key = (key << 8) | digest[i];
    return key;
}

}  // namespace host
}  // namespace vllm
