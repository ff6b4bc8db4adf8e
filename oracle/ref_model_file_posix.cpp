// POSIX stand-in for the reference's Win32-only model file reader, used ONLY to
// build the reference engine as a checker under oracle/_ref (test infrastructure).
//
// The reference declares insignia::ModelFile in include/insignia_model.hpp:20-40
// and implements it with CreateFileMappingW (src/model_file.cpp:17-44), which
// does not compile on Linux.  This file implements the same declared interface
// with open/fstat/mmap so that the rest of the reference's sources build
// unchanged.  Index format: tools/index_safetensors.py:22-34.
#include "insignia_model.hpp"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace insignia {
namespace {

struct Cursor {
    const unsigned char *p, *end;
    template <class T> T get()
    {
        if (p + sizeof(T) > end) throw std::runtime_error("bad Insignia index");
        T v;
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str(size_t n)
    {
        if (p + n > end) throw std::runtime_error("bad Insignia index");
        std::string s(reinterpret_cast<const char *>(p), n);
        p += n;
        return s;
    }
};

std::string narrow(const wchar_t *w)
{
    std::string out;
    for (; *w; ++w) out.push_back(static_cast<char>(*w)); // test paths are ASCII
    return out;
}

} // namespace

ModelFile::ModelFile(const wchar_t *index_path)
{
    const std::string path = narrow(index_path);
    FILE *f = std::fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open Insignia index");
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    std::vector<unsigned char> blob(static_cast<size_t>(n));
    const size_t got = std::fread(blob.data(), 1, blob.size(), f);
    std::fclose(f);
    if (got != blob.size()) throw std::runtime_error("cannot open Insignia index");

    Cursor c{blob.data(), blob.data() + blob.size()};
    const std::string magic = c.str(8);
    const uint32_t version = c.get<uint32_t>();
    const uint32_t count = c.get<uint32_t>();
    payload_offset_ = c.get<uint64_t>();
    if (magic != "INSIDX01" || version != 1) throw std::runtime_error("bad Insignia index");
    const uint32_t path_n = c.get<uint32_t>();
    const std::string payload = c.str(path_n);

    const int fd = ::open(payload.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("cannot open model payload");
    struct stat st {};
    if (::fstat(fd, &st) != 0) {
        ::close(fd);
        throw std::runtime_error("cannot size model payload");
    }
    mapped_bytes_ = static_cast<uint64_t>(st.st_size);
    void *m = ::mmap(nullptr, mapped_bytes_, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) throw std::runtime_error("cannot map model payload");
    mapping_ = m;
    base_ = static_cast<const std::byte *>(m);

    tensors_.reserve(count);
    for (uint32_t i = 0; i < count; i++) {
        const uint16_t name_n = c.get<uint16_t>();
        const uint8_t dtype = c.get<uint8_t>();
        const uint8_t rank = c.get<uint8_t>();
        const uint64_t off = c.get<uint64_t>();
        const uint64_t bytes = c.get<uint64_t>();
        TensorView t;
        t.name = c.str(name_n);
        t.dtype = static_cast<DType>(dtype);
        t.shape.resize(rank);
        for (auto &d : t.shape) d = c.get<uint64_t>();
        if (payload_offset_ + off + bytes > mapped_bytes_) {
            close();
            throw std::runtime_error("tensor escapes model mapping");
        }
        t.data = base_ + payload_offset_ + off;
        t.bytes = bytes;
        tensors_.push_back(std::move(t));
    }
    std::sort(tensors_.begin(), tensors_.end(), [](const TensorView &a, const TensorView &b) { return a.name < b.name; });
}

ModelFile::~ModelFile() { close(); }

ModelFile::ModelFile(ModelFile &&o) noexcept { *this = std::move(o); }

ModelFile &ModelFile::operator=(ModelFile &&o) noexcept
{
    if (this != &o) {
        close();
        file_ = o.file_;
        mapping_ = o.mapping_;
        base_ = o.base_;
        mapped_bytes_ = o.mapped_bytes_;
        payload_offset_ = o.payload_offset_;
        tensors_ = std::move(o.tensors_);
        o.file_ = o.mapping_ = nullptr;
        o.base_ = nullptr;
    }
    return *this;
}

void ModelFile::close() noexcept
{
    if (mapping_) ::munmap(mapping_, mapped_bytes_);
    mapping_ = file_ = nullptr;
    base_ = nullptr;
}

const TensorView *ModelFile::find(std::string_view name) const noexcept
{
    auto it = std::lower_bound(tensors_.begin(), tensors_.end(), name,
                               [](const TensorView &t, std::string_view n) { return t.name < n; });
    return it != tensors_.end() && it->name == name ? &*it : nullptr;
}

} // namespace insignia
