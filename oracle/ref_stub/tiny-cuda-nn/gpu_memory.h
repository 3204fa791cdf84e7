// tcnn::GPUMemory stand-in: a host vector with the same few members (host build of the test oracle).
#pragma once
#include "common.h"
namespace tcnn {
template <typename T>
class GPUMemory {
public:
    GPUMemory() {}
    explicit GPUMemory(size_t n) { resize(n); }
    void resize(size_t n) { m_bytes.assign(n * sizeof(T), 0); m_size = n; }
    void enlarge(size_t n) { if (n > m_size) resize(n); }
    void memset(int value) { std::fill(m_bytes.begin(), m_bytes.end(), (unsigned char)value); }
    T* data() { return reinterpret_cast<T*>(m_bytes.data()); }
    const T* data() const { return reinterpret_cast<const T*>(m_bytes.data()); }
    size_t size() const { return m_size; }
    size_t get_bytes() const { return m_bytes.size(); }
private:
    std::vector<unsigned char> m_bytes;
    size_t m_size = 0;
};
}  // namespace tcnn
