/*
 * Assertion and fatal-error vocabulary of the mshadow API: CHECK / CHECK_EQ... /
 * LOG(FATAL), with the same two failure modes as dmlc/mshadow's mshadow/logging.h
 * (abort by default; throw dmlc::Error when DMLC_LOG_FATAL_THROW is 1, see
 * mshadow/logging.h:183-216 there).  Written from scratch for this library.
 */
#ifndef MSHADOW_LOGGING_H_
#define MSHADOW_LOGGING_H_

#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <iostream>
#include <sstream>
#include <stdexcept>
#include <string>

#ifndef DMLC_LOG_FATAL_THROW
#define DMLC_LOG_FATAL_THROW 0
#endif

namespace dmlc {

/*! \brief exception type thrown by a failed CHECK when DMLC_LOG_FATAL_THROW is 1 */
struct Error : public std::runtime_error {
  explicit Error(const std::string &what) : std::runtime_error(what) {}
};

namespace logdetail {

inline std::string TimeStamp() {
  char buf[16];
  const time_t now = time(nullptr);
  struct tm parts;
  localtime_r(&now, &parts);
  snprintf(buf, sizeof(buf), "%02d:%02d:%02d", parts.tm_hour, parts.tm_min, parts.tm_sec);
  return buf;
}

/*! \brief collects one message; prints it to stderr when it goes out of scope */
class Line {
 public:
  Line(const char *file, int line) { text_ << "[" << TimeStamp() << "] " << file << ":" << line << ": "; }
  ~Line() { std::cerr << text_.str() << std::endl; }
  std::ostringstream &stream() { return text_; }

 private:
  std::ostringstream text_;
};

/*! \brief collects one message; aborts or throws when it goes out of scope */
class FatalLine {
 public:
  FatalLine(const char *file, int line) { text_ << "[" << TimeStamp() << "] " << file << ":" << line << ": "; }
  std::ostringstream &stream() { return text_; }
#if DMLC_LOG_FATAL_THROW
  ~FatalLine() noexcept(false) { throw Error(text_.str()); }
#else
  ~FatalLine() {
    std::cerr << text_.str() << std::endl;
    abort();
  }
#endif

 private:
  std::ostringstream text_;
};

/*! \brief lets `cond ? (void)0 : Voidify() & stream` discard the stream expression */
struct Voidify {
  void operator&(std::ostream &) {}
};

template <typename A, typename B>
inline std::string *CompareFail(const A &a, const B &b, const char *expr) {
  std::ostringstream os;
  os << "Check failed: " << expr << " (" << a << " vs. " << b << ") ";
  return new std::string(os.str());
}

}  // namespace logdetail
}  // namespace dmlc

#define LOG_INFO ::dmlc::logdetail::Line(__FILE__, __LINE__)
#define LOG_ERROR LOG_INFO
#define LOG_WARNING LOG_INFO
#define LOG_FATAL ::dmlc::logdetail::FatalLine(__FILE__, __LINE__)
#define LOG(severity) LOG_##severity.stream()
#define LOG_IF(severity, cond) \
  !(cond) ? (void)0 : ::dmlc::logdetail::Voidify() & LOG(severity)

#define CHECK(cond) \
  if (!(cond)) LOG(FATAL) << "Check failed: " #cond << ' '

#define MSHADOW_CHECK_BINARY_(a, b, op)                                                  \
  if (std::string *msh_fail_ = ((a)op(b)) ? nullptr                                      \
                                          : ::dmlc::logdetail::CompareFail((a), (b), #a " " #op " " #b)) \
  LOG(FATAL) << ::dmlc::logdetail::TakeMessage(msh_fail_)

namespace dmlc {
namespace logdetail {
inline std::string TakeMessage(std::string *m) {
  std::string s(*m);
  delete m;
  return s;
}
}  // namespace logdetail
}  // namespace dmlc

#define CHECK_EQ(a, b) MSHADOW_CHECK_BINARY_(a, b, ==)
#define CHECK_NE(a, b) MSHADOW_CHECK_BINARY_(a, b, !=)
#define CHECK_LT(a, b) MSHADOW_CHECK_BINARY_(a, b, <)
#define CHECK_LE(a, b) MSHADOW_CHECK_BINARY_(a, b, <=)
#define CHECK_GT(a, b) MSHADOW_CHECK_BINARY_(a, b, >)
#define CHECK_GE(a, b) MSHADOW_CHECK_BINARY_(a, b, >=)
#define CHECK_NOTNULL(p) \
  ((p) == nullptr ? (LOG(FATAL) << "Check notnull: " #p << ' ', (p)) : (p))

#ifdef NDEBUG
#define DCHECK(cond) while (false) CHECK(cond)
#define DCHECK_EQ(a, b) while (false) CHECK_EQ(a, b)
#define DCHECK_NE(a, b) while (false) CHECK_NE(a, b)
#define DCHECK_LT(a, b) while (false) CHECK_LT(a, b)
#define DCHECK_LE(a, b) while (false) CHECK_LE(a, b)
#define DCHECK_GT(a, b) while (false) CHECK_GT(a, b)
#define DCHECK_GE(a, b) while (false) CHECK_GE(a, b)
#else
#define DCHECK(cond) CHECK(cond)
#define DCHECK_EQ(a, b) CHECK_EQ(a, b)
#define DCHECK_NE(a, b) CHECK_NE(a, b)
#define DCHECK_LT(a, b) CHECK_LT(a, b)
#define DCHECK_LE(a, b) CHECK_LE(a, b)
#define DCHECK_GT(a, b) CHECK_GT(a, b)
#define DCHECK_GE(a, b) CHECK_GE(a, b)
#endif

#endif  // MSHADOW_LOGGING_H_
