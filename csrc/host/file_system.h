// File-system layer under the checkpoint writers and readers of the host engines.
//
// `FileSystem` is the abstract interface (create / list / size / chunked read and write / remove); `LocalFileSystem` is the
// POSIX implementation with the safety rules a checkpoint directory needs on a shared training host:
//
//   * paths: non-empty, at most 1024 bytes, no ".." component, no control characters;
//   * no component that is written to or read from may be a symbolic link (a link could redirect a privileged
//     trainer's output or feed it another user's file);
//   * a file that is read must be a regular file owned by the calling user or root, not writable by group or others,
//     and at most 1 TiB; a directory that is written to must be owned by the calling user and not writable by others;
//   * directories are created 0750, files 0640;
//   * IO goes through the descriptor in chunks of `kChunk` (32 KiB) bytes, resuming after short reads / writes and EINTR.
//
// `make_file_system(uri)` picks the implementation by scheme ("/path" or "file://path": local); other schemes are
// rejected with a clear error, so that a remote store can be added behind the same interface.
// Role in the reference: training/torch_rec_v1/torchrec_embcache/src/torchrec_embcache/csrc/file_system/file_system.h:35-58
// (interface), local_file_system/local_file_system.cpp (validation, 0750 / 0640, 32 KiB chunks), file_system_handler.cpp.
#pragma once
#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace rbh {

class FileSystem {
 public:
  static constexpr size_t kChunk = 32768;
  static constexpr long long kMaxFileBytes = 1LL << 40;
  static constexpr size_t kMaxPathBytes = 1024;
  virtual ~FileSystem() = default;
  virtual void create_dir(const std::string& dir) = 0;                       // with parents; validates every new component
  virtual bool exists(const std::string& path) const = 0;
  virtual std::vector<std::string> list_dir(const std::string& dir) const = 0;   // names, sorted
  virtual size_t file_size(const std::string& path) const = 0;
  virtual void write(const std::string& path, const void* data, size_t bytes, bool append = false) = 0;
  virtual size_t read(const std::string& path, void* out, size_t bytes, size_t offset = 0) const = 0;
  virtual void remove(const std::string& path) = 0;                          // a file or an empty directory
  std::vector<char> read_all(const std::string& path) const {
    std::vector<char> buf(file_size(path));
    if (!buf.empty() && read(path, buf.data(), buf.size(), 0) != buf.size()) throw std::runtime_error("short read: " + path);
    return buf;
  }
};

// Throws std::invalid_argument when `path` breaks one of the path rules.
inline void validate_path_text(const std::string& path) {
  if (path.empty()) throw std::invalid_argument("empty path");
  if (path.size() > FileSystem::kMaxPathBytes) throw std::invalid_argument("path longer than 1024 bytes: " + path.substr(0, 64) + "...");
  for (unsigned char c : path)
    if (c < 0x20 || c == 0x7f) throw std::invalid_argument("control character in path");
  size_t i = 0;
  while (i <= path.size()) {
    const size_t j = std::min(path.find('/', i), path.size());
    if (path.compare(i, j - i, "..") == 0) throw std::invalid_argument("'..' component in path: " + path);
    i = j + 1;
  }
}

class LocalFileSystem : public FileSystem {
 public:
  // `strict_owner` off relaxes the ownership / mode checks (not the symlink and path rules): for scratch directories of
  // tests that run as a different user than the one that created /tmp.
  explicit LocalFileSystem(bool strict_owner = true) : strict_(strict_owner) {}

  void create_dir(const std::string& dir) override {
    validate_path_text(dir);
    std::string cur;
    for (size_t i = 0; i <= dir.size(); ++i) {
      if (i == dir.size() || dir[i] == '/') {
        if (!cur.empty() && cur != "/") {
          struct stat st;
          if (::lstat(cur.c_str(), &st) == 0) {
            if (S_ISLNK(st.st_mode) && i == dir.size()) throw std::runtime_error("refusing a symbolic link as directory: " + cur);
            if (!S_ISDIR(st.st_mode) && !S_ISLNK(st.st_mode)) throw std::runtime_error("not a directory: " + cur);
          } else if (::mkdir(cur.c_str(), 0750) != 0 && errno != EEXIST) {
            throw std::runtime_error("cannot create directory " + cur + ": " + std::strerror(errno));
          }
        }
      }
      if (i < dir.size()) cur.push_back(dir[i]);
    }
  }

  bool exists(const std::string& path) const override {
    struct stat st;
    return ::lstat(path.c_str(), &st) == 0;
  }

  std::vector<std::string> list_dir(const std::string& dir) const override {
    validate_path_text(dir);
    DIR* d = ::opendir(dir.c_str());
    if (!d) throw std::runtime_error("cannot list " + dir + ": " + std::strerror(errno));
    std::vector<std::string> out;
    while (struct dirent* e = ::readdir(d)) {
      const std::string n = e->d_name;
      if (n != "." && n != "..") out.push_back(n);
    }
    ::closedir(d);
    std::sort(out.begin(), out.end());
    return out;
  }

  size_t file_size(const std::string& path) const override {
    const struct stat st = check_readable(path);
    return static_cast<size_t>(st.st_size);
  }

  void write(const std::string& path, const void* data, size_t bytes, bool append = false) override {
    validate_path_text(path);
    if (static_cast<long long>(bytes) > kMaxFileBytes) throw std::invalid_argument("write larger than 1 TiB: " + path);
    const size_t slash = path.rfind('/');
    const std::string dir = slash == std::string::npos ? "." : (slash == 0 ? "/" : path.substr(0, slash));
    check_writable_dir(dir);
    struct stat st;
    if (::lstat(path.c_str(), &st) == 0 && !S_ISREG(st.st_mode)) throw std::runtime_error("refusing to write a non-regular file: " + path);
    const int flags = O_WRONLY | O_CREAT | O_NOFOLLOW | O_CLOEXEC | (append ? O_APPEND : O_TRUNC);
    const int fd = ::open(path.c_str(), flags, 0640);
    if (fd < 0) throw std::runtime_error("cannot open for write " + path + ": " + std::strerror(errno));
    const char* p = static_cast<const char*>(data);
    size_t done = 0;
    while (done < bytes) {
      const ssize_t w = ::write(fd, p + done, std::min(kChunk, bytes - done));
      if (w < 0) {
        if (errno == EINTR) continue;
        const int e = errno;
        ::close(fd);
        throw std::runtime_error("write failed " + path + ": " + std::strerror(e));
      }
      done += static_cast<size_t>(w);
    }
    if (::close(fd) != 0) throw std::runtime_error("close failed " + path + ": " + std::strerror(errno));
  }

  size_t read(const std::string& path, void* out, size_t bytes, size_t offset = 0) const override {
    check_readable(path);
    const int fd = ::open(path.c_str(), O_RDONLY | O_NOFOLLOW | O_CLOEXEC);
    if (fd < 0) throw std::runtime_error("cannot open for read " + path + ": " + std::strerror(errno));
    char* p = static_cast<char*>(out);
    size_t done = 0;
    while (done < bytes) {
      const ssize_t r = ::pread(fd, p + done, std::min(kChunk, bytes - done), static_cast<off_t>(offset + done));
      if (r < 0) {
        if (errno == EINTR) continue;
        const int e = errno;
        ::close(fd);
        throw std::runtime_error("read failed " + path + ": " + std::strerror(e));
      }
      if (r == 0) break;        // end of file
      done += static_cast<size_t>(r);
    }
    ::close(fd);
    return done;
  }

  void remove(const std::string& path) override {
    validate_path_text(path);
    struct stat st;
    if (::lstat(path.c_str(), &st) != 0) return;
    const int rc = S_ISDIR(st.st_mode) ? ::rmdir(path.c_str()) : ::unlink(path.c_str());
    if (rc != 0) throw std::runtime_error("cannot remove " + path + ": " + std::strerror(errno));
  }

 private:
  struct stat check_readable(const std::string& path) const {
    validate_path_text(path);
    struct stat st;
    if (::lstat(path.c_str(), &st) != 0) throw std::runtime_error("no such file: " + path);
    if (S_ISLNK(st.st_mode)) throw std::invalid_argument("refusing to read through a symbolic link: " + path);
    if (!S_ISREG(st.st_mode)) throw std::invalid_argument("not a regular file: " + path);
    if (static_cast<long long>(st.st_size) > kMaxFileBytes) throw std::invalid_argument("file larger than 1 TiB: " + path);
    if (strict_) {
      if (st.st_uid != ::geteuid() && st.st_uid != 0) throw std::invalid_argument("file is owned by another user: " + path);
      if (st.st_mode & (S_IWGRP | S_IWOTH)) throw std::invalid_argument("file is writable by group or others: " + path);
    }
    if (::access(path.c_str(), R_OK) != 0) throw std::invalid_argument("no read permission: " + path);
    return st;
  }
  void check_writable_dir(const std::string& dir) const {
    struct stat st;
    if (::lstat(dir.c_str(), &st) != 0) throw std::runtime_error("no such directory: " + dir);
    if (S_ISLNK(st.st_mode)) throw std::invalid_argument("refusing to write through a symbolic link: " + dir);
    if (!S_ISDIR(st.st_mode)) throw std::invalid_argument("not a directory: " + dir);
    if (strict_) {
      if (st.st_uid != ::geteuid()) throw std::invalid_argument("directory is owned by another user: " + dir);
      if (st.st_mode & S_IWOTH) throw std::invalid_argument("directory is writable by others: " + dir);
    }
    if (::access(dir.c_str(), W_OK | X_OK) != 0) throw std::invalid_argument("no write permission: " + dir);
  }
  bool strict_;
};

// "file:///abs/path", "/abs/path" or "rel/path" -> local; any other scheme is an error.  `path_out` gets the path part.
inline std::unique_ptr<FileSystem> make_file_system(const std::string& uri, std::string* path_out = nullptr, bool strict_owner = true) {
  std::string path = uri;
  const size_t sep = uri.find("://");
  if (sep != std::string::npos) {
    const std::string scheme = uri.substr(0, sep);
    if (scheme != "file") throw std::invalid_argument("no file system registered for scheme '" + scheme + "'");
    path = uri.substr(sep + 3);
  }
  if (path_out) *path_out = path;
  return std::unique_ptr<FileSystem>(new LocalFileSystem(strict_owner));
}

}  // namespace rbh
