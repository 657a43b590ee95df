// Stand-in for yamc::barrier<> (a C++20-style cyclic thread barrier): the reference's CPU launcher constructs it with
// the number of participating threads and calls arrive_and_wait().
#pragma once
#include <cassert>
#include <condition_variable>
#include <cstddef>
#include <mutex>

namespace yamc {
template <typename CompletionFunction = void>
class barrier {
public:
    explicit barrier(std::ptrdiff_t expected) : m_expected(expected), m_waiting(0), m_generation(0) {}
    barrier(const barrier&) = delete;
    barrier& operator=(const barrier&) = delete;
    void arrive_and_wait() {
        std::unique_lock<std::mutex> lock(m_mutex);
        const std::size_t generation = m_generation;
        if (++m_waiting == m_expected) {
            m_waiting = 0;
            ++m_generation;
            m_cv.notify_all();
            return;
        }
        m_cv.wait(lock, [&] { return generation != m_generation; });
    }

private:
    std::mutex m_mutex;
    std::condition_variable m_cv;
    std::ptrdiff_t m_expected;
    std::ptrdiff_t m_waiting;
    std::size_t m_generation;
};
}  // namespace yamc
