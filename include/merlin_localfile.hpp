// LocalKVFile: keys, values and scores in three flat binary files, no header,
// host byte order -- the on-disk format of the reference's
// include/merlin_localfile.hpp:44-158, so checkpoints written by either
// implementation load in the other.
#pragma once

#include <cstdio>
#include <string>

#include "merlin/types.cuh"

namespace nv {
namespace merlin {

template <class K, class V, class S>
class LocalKVFile : public BaseKVFile<K, V, S> {
 public:
  LocalKVFile() = default;
  LocalKVFile(const LocalKVFile&) = delete;
  LocalKVFile& operator=(const LocalKVFile&) = delete;
  ~LocalKVFile() override { close(); }

  // mode is an fopen mode ("rb", "wb", "ab").  Returns false if any of the
  // three files cannot be opened.
  bool open(const std::string& keys_path, const std::string& values_path,
            const std::string& scores_path, const char* mode) {
    close();
    keys_ = std::fopen(keys_path.c_str(), mode);
    values_ = std::fopen(values_path.c_str(), mode);
    scores_ = std::fopen(scores_path.c_str(), mode);
    if (keys_ && values_ && scores_) return true;
    close();
    return false;
  }

  void close() noexcept {
    for (FILE** f : {&keys_, &values_, &scores_}) {
      if (*f) {
        std::fclose(*f);
        *f = nullptr;
      }
    }
  }

  size_t read(const size_t n, const size_t dim, K* keys, V* vectors, S* scores) override {
    const size_t got = std::fread(keys, sizeof(K), n, keys_);
    const size_t got_v = std::fread(vectors, sizeof(V) * dim, got, values_);
    const size_t got_s = std::fread(scores, sizeof(S), got, scores_);
    return (got_v == got && got_s == got) ? got : 0;
  }

  size_t write(const size_t n, const size_t dim, const K* keys, const V* vectors,
               const S* scores) override {
    const size_t put = std::fwrite(keys, sizeof(K), n, keys_);
    const size_t put_v = std::fwrite(vectors, sizeof(V) * dim, n, values_);
    const size_t put_s = std::fwrite(scores, sizeof(S), n, scores_);
    return (put == n && put_v == n && put_s == n) ? n : 0;
  }

 private:
  FILE* keys_ = nullptr;
  FILE* values_ = nullptr;
  FILE* scores_ = nullptr;
};

}  // namespace merlin
}  // namespace nv
