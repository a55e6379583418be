// Little serialiser for PODs, strings, vectors and maps with bounds-checked
// reads.  Used to keep topology / cost-model blobs in the communicator's context
// store and to move them between ranks (role of binary_stream.h in the
// reference, used for AlgResourceCtxSerializable / TopoInfo, alg_param.h:373-443
// - including the integrity checks on the way back in).
#pragma once
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <type_traits>
#include <vector>

namespace hccl {

class BinaryWriter {
public:
    template <class T>
    typename std::enable_if<std::is_trivially_copyable<T>::value, BinaryWriter&>::type operator<<(const T& v)
    {
        const uint8_t* p = reinterpret_cast<const uint8_t*>(&v);
        buf_.insert(buf_.end(), p, p + sizeof(T));
        return *this;
    }
    BinaryWriter& operator<<(const std::string& s)
    {
        *this << (uint64_t)s.size();
        buf_.insert(buf_.end(), s.begin(), s.end());
        return *this;
    }
    template <class T>
    BinaryWriter& operator<<(const std::vector<T>& v)
    {
        *this << (uint64_t)v.size();
        for (const T& e : v) *this << e;
        return *this;
    }
    template <class K, class V>
    BinaryWriter& operator<<(const std::map<K, V>& m)
    {
        *this << (uint64_t)m.size();
        for (auto& kv : m) *this << kv.first << kv.second;
        return *this;
    }
    std::vector<uint8_t> Take() { return std::move(buf_); }
    const std::vector<uint8_t>& data() const { return buf_; }

private:
    std::vector<uint8_t> buf_;
};

class BinaryReader {
public:
    explicit BinaryReader(const std::vector<uint8_t>& b) : p_(b.data()), end_(b.data() + b.size()) {}
    BinaryReader(const uint8_t* p, size_t n) : p_(p), end_(p + n) {}
    bool ok() const { return ok_; }
    bool AtEnd() const { return p_ == end_; }
    template <class T>
    typename std::enable_if<std::is_trivially_copyable<T>::value, BinaryReader&>::type operator>>(T& v)
    {
        if (!ok_ || (size_t)(end_ - p_) < sizeof(T)) { ok_ = false; return *this; }
        memcpy(&v, p_, sizeof(T));
        p_ += sizeof(T);
        return *this;
    }
    BinaryReader& operator>>(std::string& s)
    {
        uint64_t n = 0;
        *this >> n;
        if (!ok_ || n > (uint64_t)(end_ - p_)) { ok_ = false; return *this; }
        s.assign(reinterpret_cast<const char*>(p_), (size_t)n);
        p_ += n;
        return *this;
    }
    template <class T>
    BinaryReader& operator>>(std::vector<T>& v)
    {
        uint64_t n = 0;
        *this >> n;
        // an element takes at least one byte: a count beyond the remaining bytes is corrupt
        if (!ok_ || n > (uint64_t)(end_ - p_)) { ok_ = false; return *this; }
        v.clear();
        v.reserve((size_t)n);
        for (uint64_t i = 0; i < n && ok_; ++i) { T e{}; *this >> e; v.push_back(std::move(e)); }
        return *this;
    }
    template <class K, class V>
    BinaryReader& operator>>(std::map<K, V>& m)
    {
        uint64_t n = 0;
        *this >> n;
        if (!ok_ || n > (uint64_t)(end_ - p_)) { ok_ = false; return *this; }
        m.clear();
        for (uint64_t i = 0; i < n && ok_; ++i) { K k{}; V v{}; *this >> k >> v; m.emplace(std::move(k), std::move(v)); }
        return *this;
    }

private:
    const uint8_t* p_;
    const uint8_t* end_;
    bool ok_ = true;
};

}  // namespace hccl
