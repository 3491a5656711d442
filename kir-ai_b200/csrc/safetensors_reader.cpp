// Reader of the safetensors container in native code: maps a file, parses and checks its header, and hands out
// each tensor's place in the mapped payload.  A file is an 8-byte little-endian header length, a JSON header that
// maps each tensor name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to the first byte
// after the header), and the payload.  The checks are the ones of weights/safetensors_io.py (the Python reader,
// which remains as the model and as the writer) and mirror the reference's loader
// (crates/llm-backend/src/core/safetensors.rs:151-303 header, :1395-1434 per-tensor offsets; 64 MiB header cap at
// crates/llm-backend/src/core/safetensors/header.rs:3-44).
//
// Error codes: 1 model_artifact_missing, 2 model_integrity_failed, 3 unsupported_capability.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr long MAX_HEADER_BYTES = 64L * 1024 * 1024;

struct Entry {
    std::string name, dtype;
    std::vector<long> shape;
    long begin = 0, end = 0;
};

struct File {
    int fd = -1;
    void* map = nullptr;
    size_t size = 0, data_start = 0;
    std::vector<Entry> entries;
};

struct Failure {
    int code;
    std::string message;
};

int dtype_bytes(const std::string& name) {
    static const struct { const char* name; int bytes; } table[] = {
        {"F32", 4}, {"BF16", 2}, {"F16", 2}, {"F64", 8}, {"I64", 8}, {"I32", 4}, {"I16", 2}, {"I8", 1}, {"U8", 1}, {"BOOL", 1}};
    for (const auto& row : table)
        if (name == row.name) return row.bytes;
    return 0;
}

// A small JSON reader over the header: enough for objects, arrays, strings, numbers and literals.
struct Json {
    const char* p;
    const char* end;
    void skip_space() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool take(char c) {
        skip_space();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    bool string(std::string& out) {
        skip_space();
        if (p >= end || *p != '"') return false;
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            unsigned char c = (unsigned char)*p++;
            if (c < 0x20) return false;
            if (c != '\\') {
                out.push_back((char)c);
                continue;
            }
            if (p >= end) return false;
            const char e = *p++;
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    auto hex4 = [&](unsigned& v) {
                        if (end - p < 4) return false;
                        v = 0;
                        for (int i = 0; i < 4; ++i) {
                            const char h = *p++;
                            v <<= 4;
                            if (h >= '0' && h <= '9') v |= (unsigned)(h - '0');
                            else if (h >= 'a' && h <= 'f') v |= (unsigned)(h - 'a' + 10);
                            else if (h >= 'A' && h <= 'F') v |= (unsigned)(h - 'A' + 10);
                            else return false;
                        }
                        return true;
                    };
                    unsigned code = 0;
                    if (!hex4(code)) return false;
                    if (code >= 0xD800 && code <= 0xDBFF && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        unsigned low = 0;
                        if (!hex4(low)) return false;
                        if (low >= 0xDC00 && low <= 0xDFFF) code = 0x10000 + ((code - 0xD800) << 10) + (low - 0xDC00);
                    }
                    if (code < 0x80) out.push_back((char)code);
                    else if (code < 0x800) { out.push_back((char)(0xC0 | (code >> 6))); out.push_back((char)(0x80 | (code & 0x3F))); }
                    else if (code < 0x10000) {
                        out.push_back((char)(0xE0 | (code >> 12)));
                        out.push_back((char)(0x80 | ((code >> 6) & 0x3F)));
                        out.push_back((char)(0x80 | (code & 0x3F)));
                    } else {
                        out.push_back((char)(0xF0 | (code >> 18)));
                        out.push_back((char)(0x80 | ((code >> 12) & 0x3F)));
                        out.push_back((char)(0x80 | ((code >> 6) & 0x3F)));
                        out.push_back((char)(0x80 | (code & 0x3F)));
                    }
                    break;
                }
                default: return false;
            }
        }
        if (p >= end) return false;
        ++p;  // closing quote
        return true;
    }
    // A JSON integer that fits a long; false for anything else (fractions, exponents, other values).
    bool integer(long& out) {
        skip_space();
        const char* start = p;
        bool negative = false;
        if (p < end && *p == '-') { negative = true; ++p; }
        if (p >= end || *p < '0' || *p > '9') { p = start; return false; }
        unsigned long value = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (value > (unsigned long)INT64_MAX / 10) { p = start; return false; }
            value = value * 10 + (unsigned long)(*p++ - '0');
            if (value > (unsigned long)INT64_MAX) { p = start; return false; }
        }
        if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) { p = start; return false; }
        out = negative ? -(long)value : (long)value;
        return true;
    }
    bool skip_value(int depth = 0) {
        if (depth > 64) return false;
        skip_space();
        if (p >= end) return false;
        if (*p == '"') { std::string s; return string(s); }
        if (*p == '{') {
            ++p;
            if (take('}')) return true;
            do {
                std::string key;
                if (!string(key) || !take(':') || !skip_value(depth + 1)) return false;
            } while (take(','));
            return take('}');
        }
        if (*p == '[') {
            ++p;
            if (take(']')) return true;
            do {
                if (!skip_value(depth + 1)) return false;
            } while (take(','));
            return take(']');
        }
        const char* literals[] = {"true", "false", "null"};
        for (const char* word : literals) {
            const size_t n = strlen(word);
            if ((size_t)(end - p) >= n && strncmp(p, word, n) == 0) { p += n; return true; }
        }
        // a number
        const char* start = p;
        if (*p == '-') ++p;
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) ++p;
        return p > start;
    }
};

std::string describe(const std::vector<long>& shape) {
    std::string out = "[";
    for (size_t i = 0; i < shape.size(); ++i) out += (i ? ", " : "") + std::to_string(shape[i]);
    return out + "]";
}

// Whether the bytes are well-formed UTF-8 (JSON text is; a header that is not could not be handed on as names).
bool valid_utf8(const char* text, size_t length) {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(text);
    const unsigned char* end = p + length;
    while (p < end) {
        const unsigned char c = *p;
        int more;
        unsigned minimum;
        unsigned value;
        if (c < 0x80) { ++p; continue; }
        if ((c & 0xE0) == 0xC0) more = 1, minimum = 0x80, value = c & 0x1Fu;
        else if ((c & 0xF0) == 0xE0) more = 2, minimum = 0x800, value = c & 0x0Fu;
        else if ((c & 0xF8) == 0xF0) more = 3, minimum = 0x10000, value = c & 0x07u;
        else return false;
        if (end - p <= more) return false;
        for (int i = 1; i <= more; ++i) {
            if ((p[i] & 0xC0) != 0x80) return false;
            value = (value << 6) | (p[i] & 0x3Fu);
        }
        if (value < minimum || value > 0x10FFFF || (value >= 0xD800 && value <= 0xDFFF)) return false;
        p += more + 1;
    }
    return true;
}

// Parses the header into entries, checking every offset against the payload.
bool parse_header(const char* blob, size_t length, long payload_bytes, const std::string& where, std::vector<Entry>& entries,
                  Failure& failure) {
    auto broken = [&](const std::string& what) {
        failure = {2, where + ": " + what};
        return false;
    };
    if (!valid_utf8(blob, length)) return broken("header is not valid JSON");
    Json json{blob, blob + length};
    if (!json.take('{')) return broken("header must be a JSON object");
    if (!json.take('}')) {
        do {
            std::string name;
            if (!json.string(name)) return broken("header is not valid JSON");
            if (!json.take(':')) return broken("header is not valid JSON");
            if (name == "__metadata__") {
                if (!json.skip_value()) return broken("header is not valid JSON");
                continue;
            }
            if (!json.take('{')) return broken("entry `" + name + "` is not an object");
            Entry entry;
            entry.name = name;
            bool has_dtype = false, has_shape = false, has_offsets = false;
            if (!json.take('}')) {
                do {
                    std::string key;
                    if (!json.string(key) || !json.take(':')) return broken("header is not valid JSON");
                    if (key == "dtype") {
                        if (!json.string(entry.dtype)) return broken("tensor `" + name + "` has a dtype that is not a string");
                        has_dtype = true;
                    } else if (key == "shape") {
                        if (!json.take('[')) return broken("tensor `" + name + "` has a bad shape");
                        entry.shape.clear();
                        if (!json.take(']')) {
                            do {
                                long n = 0;
                                if (!json.integer(n) || n < 0) return broken("tensor `" + name + "` has a bad shape");
                                entry.shape.push_back(n);
                            } while (json.take(','));
                            if (!json.take(']')) return broken("tensor `" + name + "` has a bad shape");
                        }
                        has_shape = true;
                    } else if (key == "data_offsets") {
                        long a = 0, b = 0;
                        if (!json.take('[') || !json.integer(a) || !json.take(',') || !json.integer(b) || !json.take(']'))
                            return broken("tensor `" + name + "` has bad data_offsets");
                        entry.begin = a, entry.end = b;
                        has_offsets = true;
                    } else if (!json.skip_value()) {
                        return broken("header is not valid JSON");
                    }
                } while (json.take(','));
                if (!json.take('}')) return broken("header is not valid JSON");
            }
            if (!has_dtype) return broken("tensor `" + name + "` missing dtype");
            if (!has_shape) return broken("tensor `" + name + "` missing shape");
            if (!has_offsets) return broken("tensor `" + name + "` missing data_offsets");
            const int width = dtype_bytes(entry.dtype);
            if (width == 0) {
                failure = {3, where + ": tensor `" + name + "` has unsupported dtype " + entry.dtype};
                return false;
            }
            if (entry.begin < 0 || entry.end < entry.begin) return broken("tensor `" + name + "` has inverted data_offsets");
            if (entry.end > payload_bytes) return broken("tensor `" + name + "` data_offsets run past the payload");
            unsigned __int128 count = 1;
            for (long n : entry.shape) count *= (unsigned long)n;
            if (count * (unsigned)width != (unsigned __int128)(entry.end - entry.begin))
                return broken("tensor `" + name + "` shape " + describe(entry.shape) + " of " + entry.dtype + " does not fill its " +
                              std::to_string(entry.end - entry.begin) + " bytes");
            bool replaced = false;  // a repeated name: the last entry stands, as in a JSON object
            for (Entry& old : entries)
                if (old.name == name) {
                    old = entry;
                    replaced = true;
                }
            if (!replaced) entries.push_back(entry);
        } while (json.take(','));
        if (!json.take('}')) return broken("header is not valid JSON");
    }
    json.skip_space();
    if (json.p != json.end) return broken("header is not valid JSON");
    if (entries.empty()) return broken("file holds no tensors");
    return true;
}

void report(const Failure& failure, int* code, char* message, int capacity) {
    if (code) *code = failure.code;
    if (message && capacity > 0) {
        snprintf(message, (size_t)capacity, "%s", failure.message.c_str());
    }
}

}  // namespace

#define KIRAI_HOST_EXPORT extern "C" __attribute__((visibility("default")))

// Maps the file and reads its header.  Returns a handle, or null with `code` and `message` set.
KIRAI_HOST_EXPORT void* kirai_st_open(const char* path, int* code, char* message, int capacity) {
    const std::string where = path ? path : "";
    auto fail = [&](int c, const std::string& what) -> void* {
        report({c, where + ": " + what}, code, message, capacity);
        return nullptr;
    };
    const int fd = path ? open(path, O_RDONLY) : -1;
    if (fd < 0) return fail(1, "no such file");
    struct stat info;
    if (fstat(fd, &info) != 0 || info.st_size < 8) {
        close(fd);
        return fail(2, "missing the 8-byte header length");
    }
    const size_t size = (size_t)info.st_size;
    void* map = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return fail(2, "the file cannot be mapped");
    }
    const unsigned char* bytes = static_cast<const unsigned char*>(map);
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | bytes[i];
    Failure failure{0, ""};
    File* file = nullptr;
    if (header_len > (uint64_t)MAX_HEADER_BYTES) failure = {2, where + ": header of " + std::to_string(header_len) + " bytes exceeds 64 MiB"};
    else if (8 + header_len > size) failure = {2, where + ": header runs past the end of the file"};
    else {
        file = new File();
        file->fd = fd, file->map = map, file->size = size, file->data_start = 8 + (size_t)header_len;
        if (!parse_header(reinterpret_cast<const char*>(bytes) + 8, (size_t)header_len, (long)(size - file->data_start), where,
                          file->entries, failure)) {
            delete file;
            file = nullptr;
        }
    }
    if (!file) {
        munmap(map, size);
        close(fd);
        report(failure, code, message, capacity);
        return nullptr;
    }
    if (code) *code = 0;
    return file;
}

KIRAI_HOST_EXPORT void kirai_st_close(void* handle) {
    File* file = static_cast<File*>(handle);
    if (!file) return;
    munmap(file->map, file->size);
    close(file->fd);
    delete file;
}

KIRAI_HOST_EXPORT int kirai_st_count(void* handle) { return (int)static_cast<File*>(handle)->entries.size(); }

// Entry `index`: name and dtype as C strings (-8 if a buffer is too small), shape (rank <= 16), byte range.
KIRAI_HOST_EXPORT int kirai_st_entry(void* handle, int index, char* name, int name_capacity, char* dtype, int dtype_capacity,
                                     long* shape, int* rank, long* begin, long* end) {
    File* file = static_cast<File*>(handle);
    if (index < 0 || index >= (int)file->entries.size()) return -6;
    const Entry& entry = file->entries[(size_t)index];
    if ((int)entry.name.size() + 1 > name_capacity || (int)entry.dtype.size() + 1 > dtype_capacity || entry.shape.size() > 16) return -8;
    memcpy(name, entry.name.c_str(), entry.name.size() + 1);
    memcpy(dtype, entry.dtype.c_str(), entry.dtype.size() + 1);
    for (size_t i = 0; i < entry.shape.size(); ++i) shape[i] = entry.shape[i];
    *rank = (int)entry.shape.size();
    *begin = entry.begin;
    *end = entry.end;
    return 0;
}

// The first byte of the payload in the mapping (read-only memory) and its length.
KIRAI_HOST_EXPORT const void* kirai_st_payload(void* handle) {
    File* file = static_cast<File*>(handle);
    return static_cast<const char*>(file->map) + file->data_start;
}
KIRAI_HOST_EXPORT long kirai_st_payload_bytes(void* handle) {
    File* file = static_cast<File*>(handle);
    return (long)(file->size - file->data_start);
}
