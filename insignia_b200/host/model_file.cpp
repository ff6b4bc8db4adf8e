// POSIX implementation of insignia::ModelFile (interface: include/insignia_model.hpp;
// reference behaviour: src/model_file.cpp:17-44, format: tools/index_safetensors.py:22-34).
#include "insignia_model.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <stdexcept>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace insignia {
namespace {

// Bounds-checked little-endian reader over the index blob.
class Reader {
public:
    Reader(const unsigned char *p, size_t n) : p_(p), end_(p + n) {}
    template <class T> T pod()
    {
        need(sizeof(T));
        T v;
        std::memcpy(&v, p_, sizeof(T));
        p_ += sizeof(T);
        return v;
    }
    std::string text(size_t n)
    {
        need(n);
        std::string s(reinterpret_cast<const char *>(p_), n);
        p_ += n;
        return s;
    }

private:
    void need(size_t n) const
    {
        if (size_t(end_ - p_) < n) throw std::runtime_error("bad Insignia index");
    }
    const unsigned char *p_, *end_;
};

std::vector<unsigned char> slurp(const std::string &path)
{
    FILE *f = std::fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open Insignia index");
    std::vector<unsigned char> blob;
    unsigned char buf[1 << 16];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof(buf), f)) > 0) blob.insert(blob.end(), buf, buf + n);
    std::fclose(f);
    return blob;
}

} // namespace

ModelFile::ModelFile(const wchar_t *index_path)
{
    std::string narrow;
    for (const wchar_t *p = index_path; p && *p; ++p) {
        // UTF-8 encode the code point (paths in practice are ASCII)
        const uint32_t c = static_cast<uint32_t>(*p);
        if (c < 0x80) narrow.push_back(char(c));
        else if (c < 0x800) { narrow.push_back(char(0xC0 | (c >> 6))); narrow.push_back(char(0x80 | (c & 0x3F))); }
        else if (c < 0x10000) { narrow.push_back(char(0xE0 | (c >> 12))); narrow.push_back(char(0x80 | ((c >> 6) & 0x3F))); narrow.push_back(char(0x80 | (c & 0x3F))); }
        else { narrow.push_back(char(0xF0 | (c >> 18))); narrow.push_back(char(0x80 | ((c >> 12) & 0x3F))); narrow.push_back(char(0x80 | ((c >> 6) & 0x3F))); narrow.push_back(char(0x80 | (c & 0x3F))); }
    }
    open(narrow);
}

ModelFile::ModelFile(const char *index_path) { open(index_path ? index_path : ""); }

void ModelFile::open(const std::string &index_path)
{
    const std::vector<unsigned char> blob = slurp(index_path);
    Reader r(blob.data(), blob.size());
    const std::string magic = r.text(8);
    const uint32_t version = r.pod<uint32_t>();
    const uint32_t count = r.pod<uint32_t>();
    const uint64_t payload = r.pod<uint64_t>();
    if (magic != "INSIDX01" || version != 1) throw std::runtime_error("bad Insignia index");
    payload_offset_ = payload;
    const std::string payload_path = r.text(r.pod<uint32_t>());

    const int fd = ::open(payload_path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) throw std::runtime_error("cannot open model payload");
    struct stat st {};
    if (::fstat(fd, &st) != 0) {
        ::close(fd);
        throw std::runtime_error("cannot size model payload");
    }
    mapped_bytes_ = uint64_t(st.st_size);
    void *m = mapped_bytes_ ? ::mmap(nullptr, mapped_bytes_, PROT_READ, MAP_PRIVATE, fd, 0) : MAP_FAILED;
    ::close(fd); // the mapping keeps the file alive
    if (m == MAP_FAILED) {
        mapped_bytes_ = 0;
        throw std::runtime_error("cannot map model payload");
    }
    mapping_ = m;
    base_ = static_cast<const std::byte *>(m);

    try {
        tensors_.reserve(count);
        for (uint32_t i = 0; i < count; i++) {
            const uint16_t name_n = r.pod<uint16_t>();
            const uint8_t dtype = r.pod<uint8_t>();
            const uint8_t rank = r.pod<uint8_t>();
            const uint64_t off = r.pod<uint64_t>();
            const uint64_t bytes = r.pod<uint64_t>();
            TensorView t;
            t.name = r.text(name_n);
            t.dtype = static_cast<DType>(dtype);
            t.shape.resize(rank);
            for (uint64_t &d : t.shape) d = r.pod<uint64_t>();
            if (payload_offset_ + off + bytes > mapped_bytes_ || payload_offset_ + off + bytes < bytes)
                throw std::runtime_error("tensor escapes model mapping");
            t.data = base_ + payload_offset_ + off;
            t.bytes = bytes;
            tensors_.push_back(std::move(t));
        }
    } catch (...) {
        close();
        tensors_.clear();
        throw;
    }
    std::sort(tensors_.begin(), tensors_.end(), [](const TensorView &a, const TensorView &b) { return a.name < b.name; });
}

ModelFile::~ModelFile() { close(); }

ModelFile::ModelFile(ModelFile &&other) noexcept { *this = std::move(other); }

ModelFile &ModelFile::operator=(ModelFile &&other) noexcept
{
    if (this != &other) {
        close();
        mapping_ = other.mapping_;
        base_ = other.base_;
        mapped_bytes_ = other.mapped_bytes_;
        payload_offset_ = other.payload_offset_;
        tensors_ = std::move(other.tensors_);
        other.mapping_ = nullptr;
        other.base_ = nullptr;
        other.mapped_bytes_ = 0;
        other.tensors_.clear();
    }
    return *this;
}

void ModelFile::close() noexcept
{
    if (mapping_) ::munmap(mapping_, mapped_bytes_);
    mapping_ = nullptr;
    base_ = nullptr;
}

const TensorView *ModelFile::find(std::string_view name) const noexcept
{
    size_t lo = 0, hi = tensors_.size();
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (std::string_view(tensors_[mid].name) < name) lo = mid + 1;
        else hi = mid;
    }
    return lo < tensors_.size() && tensors_[lo].name == name ? &tensors_[lo] : nullptr;
}

} // namespace insignia
