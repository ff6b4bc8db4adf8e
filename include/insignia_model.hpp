// Model file: zero-copy view of a safetensors payload through an INSIDX01 index.
//
// Drop-in for the reference header of the same name (include/insignia_model.hpp:10-40):
// same namespace, types, members and error strings, implemented with POSIX
// open/fstat/mmap instead of Win32 file mappings.  Index format:
// tools/index_safetensors.py:22-34; reader contract: src/model_file.cpp:17-44.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <string_view>
#include <vector>

#if defined(__GNUC__)
#define INSIGNIA_API __attribute__((visibility("default")))
#else
#define INSIGNIA_API
#endif

namespace insignia {

// Codes as written by the index builder (tools/index_safetensors.py:8).
enum class DType : uint8_t { f32 = 1, bf16 = 2, f16 = 3, u8 = 4, u32 = 5, i8 = 6 };

struct TensorView {
    std::string name;
    DType dtype{};
    std::vector<uint64_t> shape;
    const std::byte *data{}; // inside the mapping; valid while the ModelFile lives
    uint64_t bytes{};
};

class INSIGNIA_API ModelFile final {
public:
    ModelFile() = default;
    // Wide path as in the reference (its drivers pass wmain's argv); narrowed byte-wise on POSIX.
    explicit ModelFile(const wchar_t *index_path);
    // Additive: UTF-8 path.
    explicit ModelFile(const char *index_path);
    ~ModelFile();
    ModelFile(const ModelFile &) = delete;
    ModelFile &operator=(const ModelFile &) = delete;
    ModelFile(ModelFile &&other) noexcept;
    ModelFile &operator=(ModelFile &&other) noexcept;

    // Binary search over the name-sorted table; nullptr when absent.
    const TensorView *find(std::string_view name) const noexcept;
    const std::vector<TensorView> &tensors() const noexcept { return tensors_; }
    uint64_t payload_offset() const noexcept { return payload_offset_; }

private:
    void open(const std::string &index_path);
    void close() noexcept;
    void *mapping_{};
    const std::byte *base_{};
    uint64_t mapped_bytes_{};
    uint64_t payload_offset_{};
    std::vector<TensorView> tensors_;
};

} // namespace insignia
