// Weight archives of the reference (".ct" files): dl::io::save / dl::io::load.
//
// Layout (src/io/checkpoint.cpp:17,52-114 and src/io/archive.h:14-30 of the reference), every integer little-endian:
//     8 bytes   'C','T','O','R','C','H',0,1
//     u64       number of entries
//     per entry u64 name length, the name's bytes,
//               u8 dtype (f32 0, f64 1, i64 2, bool 3, f16 4, bf16 5), u64 rank, rank x u64 extents,
//               the elements, dense row-major, little-endian scalars
// Tensors are read to host memory; Module::load_state_dict moves them to the module's device.  Writing goes to a
// temporary file beside the target that is renamed over it when complete, so a failed save leaves the old file.
#include "dl/dl.h"

#include <array>
#include <bit>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <limits>
#include <stdexcept>

namespace dl::io {

namespace {

constexpr std::array<unsigned char, 8> kMagic{'C', 'T', 'O', 'R', 'C', 'H', 0, 1};
static_assert(std::endian::native == std::endian::little, "the archive code assumes a little-endian host (x86-64, aarch64)");

void put_u64(std::ostream& out, std::uint64_t value) {
    unsigned char bytes[8];
    for (int i = 0; i < 8; ++i) bytes[i] = static_cast<unsigned char>(value >> (8 * i));
    out.write(reinterpret_cast<const char*>(bytes), 8);
}

std::uint64_t get_u64(std::istream& in) {
    unsigned char bytes[8];
    in.read(reinterpret_cast<char*>(bytes), 8);
    std::uint64_t value = 0;
    for (int i = 0; i < 8; ++i) value |= static_cast<std::uint64_t>(bytes[i]) << (8 * i);
    return value;
}

}  // namespace

void save(const std::filesystem::path& path, std::span<const NamedTensor> state) {
    std::filesystem::path scratch = path;
    scratch += ".partial";
    {
        std::ofstream out;
        out.exceptions(std::ios::failbit | std::ios::badbit);
        out.open(scratch, std::ios::binary | std::ios::trunc);
        out.write(reinterpret_cast<const char*>(kMagic.data()), kMagic.size());
        put_u64(out, state.size());
        for (const auto& [name, tensor] : state) {
            if (!tensor.defined()) throw std::invalid_argument("state entry '" + name + "' holds no tensor");
            put_u64(out, name.size());
            out.write(name.data(), static_cast<std::streamsize>(name.size()));
            out.put(static_cast<char>(tensor.dtype()));
            put_u64(out, static_cast<std::uint64_t>(tensor.ndim()));
            for (Index extent : tensor.shape()) put_u64(out, static_cast<std::uint64_t>(extent));
            const Tensor host = tensor.to(Device::cpu());   // tensors of this library are always dense row-major
            out.write(static_cast<const char*>(host.raw_data()), static_cast<std::streamsize>(host.nbytes()));
        }
        out.flush();
    }
    std::filesystem::rename(scratch, path);
}

StateDict load(const std::filesystem::path& path) {
    std::ifstream in;
    in.exceptions(std::ios::failbit | std::ios::badbit | std::ios::eofbit);
    in.open(path, std::ios::binary);
    const auto file_bytes = std::filesystem::file_size(path);
    std::array<unsigned char, 8> magic{};
    in.read(reinterpret_cast<char*>(magic.data()), magic.size());
    if (magic != kMagic) throw std::runtime_error("unsupported Ctorch checkpoint format");
    const std::uint64_t count = get_u64(in);
    if (count > file_bytes) throw std::runtime_error("corrupt Ctorch checkpoint: entry count exceeds the file size");
    StateDict result;
    result.reserve(static_cast<std::size_t>(count));
    for (std::uint64_t entry = 0; entry < count; ++entry) {
        const std::uint64_t name_bytes = get_u64(in);
        if (name_bytes > file_bytes) throw std::runtime_error("corrupt Ctorch checkpoint: name length exceeds the file size");
        std::string name(static_cast<std::size_t>(name_bytes), '\0');
        in.read(name.data(), static_cast<std::streamsize>(name_bytes));
        const int code = in.get();
        if (code < 0 || code > static_cast<int>(DType::bf16)) throw std::runtime_error("corrupt Ctorch checkpoint: unknown dtype in '" + name + "'");
        const auto dtype = static_cast<DType>(code);
        const std::uint64_t rank = get_u64(in);
        if (rank > 64) throw std::runtime_error("corrupt Ctorch checkpoint: rank of '" + name + "'");
        Shape shape(static_cast<std::size_t>(rank));
        std::uint64_t elements = 1;
        for (auto& extent : shape) {
            const std::uint64_t value = get_u64(in);
            if (value > file_bytes || (value != 0 && elements > file_bytes / value + 1))
                throw std::runtime_error("corrupt Ctorch checkpoint: extents of '" + name + "' exceed the file size");
            elements *= value;
            extent = static_cast<Index>(value);
        }
        if (elements * element_size(dtype) > file_bytes) throw std::runtime_error("corrupt Ctorch checkpoint: '" + name + "' exceeds the file size");
        Tensor tensor = empty(shape, TensorOptions{dtype, Device::cpu()});
        in.read(static_cast<char*>(tensor.mutable_data()), static_cast<std::streamsize>(tensor.nbytes()));
        result.emplace_back(std::move(name), std::move(tensor));
    }
    return result;
}

}  // namespace dl::io
