// Bounds-checked reader for the FlatBuffers `Graph` file (reference schema/graph.fbs:1-68).
//
// The reference links flatc-generated accessors (csrc/runtime/execution_engine.cpp:25,
// `fxfusion::GetGraph`).  This reader walks the same binary encoding directly: a root
// uoffset, tables whose first word is the signed distance back to their vtable, vtables of
// u16 field offsets indexed by field id (0 = field absent, use the schema default), vectors
// as a u32 count followed by the elements, strings as a u32 length plus bytes.
// Every dereference is checked against the buffer length so that a truncated or corrupt
// file yields an error message instead of a wild read.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

namespace fxf {
namespace fbs {

struct Buffer {
    const uint8_t* data = nullptr;
    size_t size = 0;
    void need(size_t pos, size_t n, const char* what) const {
        if (pos > size || n > size - pos) throw std::runtime_error(std::string("graph file corrupt: ") + what + " out of bounds");
    }
    template <typename T> T read(size_t pos, const char* what) const {
        need(pos, sizeof(T), what);
        T v;
        std::memcpy(&v, data + pos, sizeof(T));
        return v;
    }
};

template <typename T> struct Span {
    const uint8_t* base = nullptr;
    uint32_t count = 0;
    uint32_t size() const { return count; }
    T operator[](uint32_t i) const {
        T v;
        std::memcpy(&v, base + sizeof(T) * size_t(i), sizeof(T));
        return v;
    }
};

class Table {
public:
    Table() = default;
    Table(const Buffer* b, size_t pos) : b_(b), pos_(pos) {
        int32_t soff = b_->read<int32_t>(pos, "table");
        int64_t vt = int64_t(pos) - int64_t(soff);
        if (vt < 0) throw std::runtime_error("graph file corrupt: vtable before start of file");
        vt_ = size_t(vt);
        vt_size_ = b_->read<uint16_t>(vt_, "vtable");
        if (vt_size_ < 4) throw std::runtime_error("graph file corrupt: vtable too small");
        b_->need(vt_, vt_size_, "vtable");
    }
    bool valid() const { return b_ != nullptr; }

    template <typename T> T scalar(int field, T def) const {
        size_t p = field_pos(field);
        return p ? b_->read<T>(p, "scalar field") : def;
    }
    template <typename T> Span<T> vec(int field) const {
        size_t p = indirect(field);
        Span<T> s;
        if (!p) return s;
        uint32_t n = b_->read<uint32_t>(p, "vector length");
        b_->need(p + 4, size_t(n) * sizeof(T), "vector payload");
        s.base = b_->data + p + 4;
        s.count = n;
        return s;
    }
    std::string str(int field) const {
        size_t p = indirect(field);
        if (!p) return std::string();
        uint32_t n = b_->read<uint32_t>(p, "string length");
        b_->need(p + 4, n, "string payload");
        return std::string(reinterpret_cast<const char*>(b_->data + p + 4), n);
    }
    uint32_t table_vec_size(int field) const {
        size_t p = indirect(field);
        if (!p) return 0;
        uint32_t n = b_->read<uint32_t>(p, "vector length");
        b_->need(p + 4, size_t(n) * 4, "vector payload");
        return n;
    }
    Table table_at(int field, uint32_t i) const {
        size_t p = indirect(field);
        size_t slot = p + 4 + size_t(i) * 4;
        uint32_t rel = b_->read<uint32_t>(slot, "table reference");
        return Table(b_, slot + rel);
    }

private:
    size_t field_pos(int field) const {
        size_t slot = 4 + 2 * size_t(field);
        if (slot + 2 > vt_size_) return 0;
        uint16_t rel = b_->read<uint16_t>(vt_ + slot, "vtable slot");
        return rel ? pos_ + rel : 0;
    }
    size_t indirect(int field) const {
        size_t p = field_pos(field);
        if (!p) return 0;
        uint32_t rel = b_->read<uint32_t>(p, "reference field");
        b_->need(p, rel, "reference target");
        return p + rel;
    }
    const Buffer* b_ = nullptr;
    size_t pos_ = 0, vt_ = 0;
    uint16_t vt_size_ = 0;
};

inline Table root(const Buffer* b) {
    uint32_t off = b->read<uint32_t>(0, "root offset");
    return Table(b, off);
}

// Field ids, in schema declaration order.
namespace GraphF { enum { name = 0, arena_size = 1, tensors = 2, nodes = 3 }; }
namespace TensorF { enum { id = 0, kind = 1, offset = 2, size_bytes = 3, shape = 4, dtype = 5, alias_of = 6, data = 7 }; }
namespace NodeF { enum { op_code = 0, input_ids = 1, output_ids = 2, int_params = 3, float_params = 4 }; }

}  // namespace fbs
}  // namespace fxf
