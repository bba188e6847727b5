// Reader of the safetensors format: maps a file, parses and checks its header, and hands out the
// tensors' places in the map; a copy routine moves a tensor's bytes out with several threads, which
// is what loading a checkpoint of several gigabytes spends its time on (page faults of the map).
//
// Format: 8 bytes little-endian header length N, N bytes of JSON mapping each tensor name to
// {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]} with offsets counted from the end
// of the header ("__metadata__" maps strings to strings), then the raw little-endian data.
//
// Every entry point returns 0 or a negative code and, where it takes `err`, writes a message that
// names the file and the tensor.  Nothing here touches the GPU.
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <thread>
#include <vector>

#define DFI_IO_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct Entry {
    std::string name, dtype;
    std::vector<long long> shape;
    long long begin = 0, end = 0;
};

struct File {
    std::string path;
    int fd = -1;
    unsigned char* map = nullptr;
    long long size = 0, data_start = 0;
    std::vector<Entry> entries;
    std::string metadata;      // the JSON text of "__metadata__" (an object) or empty
};

int element_size(const std::string& dtype) {
    if (dtype == "F64" || dtype == "I64" || dtype == "U64") return 8;
    if (dtype == "F32" || dtype == "I32" || dtype == "U32") return 4;
    if (dtype == "F16" || dtype == "BF16" || dtype == "I16" || dtype == "U16") return 2;
    if (dtype == "I8" || dtype == "U8" || dtype == "BOOL" || dtype == "F8_E4M3" || dtype == "F8_E5M2") return 1;
    return 0;
}

// A parser for the header's JSON: objects, arrays, strings, integers; anything else is an error.
struct Parser {
    const char* p;
    const char* end;
    std::string error;

    void skip() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool fail(const char* what) {
        if (error.empty()) error = what;
        return false;
    }
    bool expect(char c) {
        skip();
        if (p < end && *p == c) { ++p; return true; }
        return fail("header is not valid JSON");
    }
    bool peek(char c) {
        skip();
        return p < end && *p == c;
    }
    static void utf8(std::string& out, unsigned code) {
        if (code < 0x80) out += (char)code;
        else if (code < 0x800) { out += (char)(0xC0 | (code >> 6)); out += (char)(0x80 | (code & 0x3F)); }
        else if (code < 0x10000) {
            out += (char)(0xE0 | (code >> 12)); out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F));
        } else {
            out += (char)(0xF0 | (code >> 18)); out += (char)(0x80 | ((code >> 12) & 0x3F));
            out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F));
        }
    }
    bool hex4(unsigned& code) {
        if (end - p < 4) return fail("header is not valid JSON");
        code = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p++;
            code <<= 4;
            if (c >= '0' && c <= '9') code |= (unsigned)(c - '0');
            else if (c >= 'a' && c <= 'f') code |= (unsigned)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') code |= (unsigned)(c - 'A' + 10);
            else return fail("header is not valid JSON");
        }
        return true;
    }
    bool string(std::string& out) {
        out.clear();
        if (!expect('"')) return false;
        while (p < end && *p != '"') {
            if (*p != '\\') { out += *p++; continue; }
            if (++p >= end) break;
            const char c = *p++;
            switch (c) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned code = 0;
                    if (!hex4(code)) return false;
                    if (code >= 0xD800 && code < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        unsigned low = 0;
                        if (!hex4(low)) return false;
                        code = 0x10000 + ((code - 0xD800) << 10) + (low - 0xDC00);
                    }
                    utf8(out, code);
                    break;
                }
                default: return fail("header is not valid JSON");
            }
        }
        if (p >= end) return fail("header is not valid JSON");
        ++p;
        return true;
    }
    bool integer(long long& out) {
        skip();
        const char* start = p;
        bool negative = false;
        if (p < end && *p == '-') { negative = true; ++p; }
        unsigned long long v = 0;
        const char* digits = p;
        while (p < end && *p >= '0' && *p <= '9') {
            if (v > 900000000000000000ULL) return fail("header holds a number that is too large");
            v = v * 10 + (unsigned)(*p++ - '0');
        }
        if (p == digits || p == start) return fail("header is not valid JSON");
        out = negative ? -(long long)v : (long long)v;
        return true;
    }
    bool integers(std::vector<long long>& out) {
        out.clear();
        if (!expect('[')) return false;
        if (peek(']')) { ++p; return true; }
        for (;;) {
            long long v = 0;
            if (!integer(v)) return false;
            out.push_back(v);
            if (peek(',')) { ++p; continue; }
            return expect(']');
        }
    }
    // skips one value of any kind and returns its text span (used for "__metadata__")
    bool any(const char*& from, const char*& to) {
        skip();
        from = p;
        if (p >= end) return fail("header is not valid JSON");
        if (*p == '"') { std::string s; if (!string(s)) return false; }
        else if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            ++p;
            if (peek(close)) { ++p; to = p; return true; }
            for (;;) {
                if (open == '{') {
                    std::string key;
                    if (!string(key) || !expect(':')) return false;
                }
                const char *a, *b;
                if (!any(a, b)) return false;
                if (peek(',')) { ++p; continue; }
                if (!expect(close)) return false;
                break;
            }
        } else {
            while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') ++p;
            if (p == from) return fail("header is not valid JSON");
        }
        to = p;
        return true;
    }
};

bool parse_header(File& f, const char* text, long long length, std::string& error) {
    Parser ps{text, text + length, {}};
    if (!ps.expect('{')) { error = ps.error; return false; }
    if (ps.peek('}')) return true;
    for (;;) {
        std::string name;
        if (!ps.string(name) || !ps.expect(':')) { error = ps.error; return false; }
        if (name == "__metadata__") {
            const char *a, *b;
            if (!ps.any(a, b)) { error = ps.error; return false; }
            f.metadata.assign(a, b);
        } else {
            Entry e;
            e.name = name;
            bool has_dtype = false, has_shape = false, has_offsets = false;
            if (!ps.expect('{')) { error = ps.error; return false; }
            if (!ps.peek('}')) {
                for (;;) {
                    std::string key;
                    if (!ps.string(key) || !ps.expect(':')) { error = ps.error; return false; }
                    if (key == "dtype") {
                        if (!ps.string(e.dtype)) { error = ps.error; return false; }
                        has_dtype = true;
                    } else if (key == "shape") {
                        if (!ps.integers(e.shape)) { error = ps.error; return false; }
                        has_shape = true;
                    } else if (key == "data_offsets") {
                        std::vector<long long> two;
                        if (!ps.integers(two)) { error = ps.error; return false; }
                        if (two.size() != 2) { error = "tensor '" + name + "' has data_offsets that are not a pair"; return false; }
                        e.begin = two[0];
                        e.end = two[1];
                        has_offsets = true;
                    } else {
                        const char *a, *b;
                        if (!ps.any(a, b)) { error = ps.error; return false; }
                    }
                    if (ps.peek(',')) { ++ps.p; continue; }
                    break;
                }
            }
            if (!ps.expect('}')) { error = ps.error; return false; }
            if (!has_dtype || !has_shape || !has_offsets) {
                error = "tensor '" + name + "' lacks dtype, shape or data_offsets";
                return false;
            }
            f.entries.push_back(e);
        }
        if (ps.peek(',')) { ++ps.p; continue; }
        if (!ps.expect('}')) { error = ps.error; return false; }
        return true;
    }
}

void put(char* err, int err_len, const std::string& message) {
    if (err == nullptr || err_len <= 0) return;
    snprintf(err, (size_t)err_len, "%s", message.c_str());
}

void release(File* f) {
    if (f->map != nullptr) munmap(f->map, (size_t)f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

}  // namespace

// Opens and checks a file.  On failure *out stays null and err says why.
DFI_IO_EXPORT int dfi_st_open(const char* path, void** out, char* err, int err_len) {
    *out = nullptr;
    File* f = new File;
    f->path = path;
    f->fd = open(path, O_RDONLY);
    struct stat st;
    if (f->fd < 0 || fstat(f->fd, &st) != 0) {
        put(err, err_len, f->path + ": cannot be opened");
        release(f);
        return -1;
    }
    f->size = (long long)st.st_size;
    if (f->size < 8) {
        put(err, err_len, f->path + ": truncated (no header length)");
        release(f);
        return -2;
    }
    void* map = mmap(nullptr, (size_t)f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (map == MAP_FAILED) {
        put(err, err_len, f->path + ": cannot be mapped");
        release(f);
        return -1;
    }
    f->map = (unsigned char*)map;
    unsigned long long n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | f->map[i];
    if (n > (unsigned long long)(f->size - 8)) {
        put(err, err_len, f->path + ": truncated (header of " + std::to_string(n) + " bytes, file of " + std::to_string(f->size) + ")");
        release(f);
        return -2;
    }
    f->data_start = 8 + (long long)n;
    std::string why;
    if (!parse_header(*f, (const char*)f->map + 8, (long long)n, why)) {
        put(err, err_len, f->path + ": " + why);
        release(f);
        return -3;
    }
    for (const Entry& e : f->entries) {
        const int width = element_size(e.dtype);
        if (width == 0) {
            put(err, err_len, f->path + ": tensor '" + e.name + "' has unsupported dtype " + e.dtype);
            release(f);
            return -4;
        }
        long long count = 1;
        for (long long s : e.shape) {
            if (s < 0 || (s > 0 && count > (1LL << 56) / s)) {
                put(err, err_len, f->path + ": tensor '" + e.name + "' has a shape that is not a size");
                release(f);
                return -4;
            }
            count *= s;
        }
        if (e.begin < 0 || e.end < e.begin || e.end - e.begin != count * width) {
            put(err, err_len, f->path + ": tensor '" + e.name + "' spans " + std::to_string(e.end - e.begin) +
                                  " bytes, shape needs " + std::to_string(count * width));
            release(f);
            return -4;
        }
        if (f->data_start + e.end > f->size) {
            put(err, err_len, f->path + ": truncated (tensor '" + e.name + "' ends past the file)");
            release(f);
            return -2;
        }
    }
    *out = f;
    return 0;
}

DFI_IO_EXPORT void dfi_st_close(void* handle) {
    if (handle != nullptr) release((File*)handle);
}

DFI_IO_EXPORT int dfi_st_count(void* handle) { return (int)((File*)handle)->entries.size(); }

// Entry i: pointers stay valid until the file is closed.  `shape` gets up to `max_dims` sizes.
DFI_IO_EXPORT int dfi_st_entry(void* handle, int i, const char** name, const char** dtype, int* n_dims, long long* shape,
                               int max_dims, long long* begin, long long* end) {
    File* f = (File*)handle;
    if (i < 0 || i >= (int)f->entries.size()) return -1;
    const Entry& e = f->entries[(size_t)i];
    if ((int)e.shape.size() > max_dims) return -2;
    *name = e.name.c_str();
    *dtype = e.dtype.c_str();
    *n_dims = (int)e.shape.size();
    for (size_t d = 0; d < e.shape.size(); ++d) shape[d] = e.shape[d];
    *begin = e.begin;
    *end = e.end;
    return 0;
}

// The text of "__metadata__" (a JSON object) and its length; null when the header has none.
DFI_IO_EXPORT const char* dfi_st_metadata(void* handle, long long* length) {
    File* f = (File*)handle;
    *length = (long long)f->metadata.size();
    return f->metadata.empty() ? nullptr : f->metadata.c_str();
}

// Start of the data section in the map, and its size.
DFI_IO_EXPORT const unsigned char* dfi_st_data(void* handle, long long* size) {
    File* f = (File*)handle;
    *size = f->size - f->data_start;
    return f->map + f->data_start;
}

// Copies bytes [begin, begin + n_bytes) of the data section to dst with up to `threads` threads.
DFI_IO_EXPORT int dfi_st_read(void* handle, long long begin, long long n_bytes, void* dst, int threads) {
    File* f = (File*)handle;
    if (begin < 0 || n_bytes < 0 || f->data_start + begin + n_bytes > f->size) return -1;
    const unsigned char* src = f->map + f->data_start + begin;
    const long long chunk = 8LL << 20;
    int n = (int)((n_bytes + chunk - 1) / chunk);
    if (n > threads) n = threads;
    if (n <= 1) {
        memcpy(dst, src, (size_t)n_bytes);
        return 0;
    }
    std::vector<std::thread> pool;
    const long long per = ((n_bytes / n) + 4095) & ~4095LL;
    for (int t = 0; t < n; ++t) {
        const long long from = per * t;
        if (from >= n_bytes) break;
        const long long len = (from + per > n_bytes) ? n_bytes - from : per;
        pool.emplace_back([=] { memcpy((unsigned char*)dst + from, src + from, (size_t)len); });
    }
    for (std::thread& th : pool) th.join();
    return 0;
}
