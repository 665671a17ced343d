#include "Logger.h"

#include <chrono>
#include <ctime>
#include <iomanip>
#include <iostream>
#include <sstream>

Logger logger;

Logger::Logger(const std::string& filePath, bool c, bool f) : log2Console(c), log2File(f && !filePath.empty()) {
    if (log2File) logFile.open(filePath, std::ios::app);
}

Logger::~Logger() {
    if (logFile.is_open()) logFile.close();
}

std::string Logger::getTimeStamp() {
    auto now = std::chrono::system_clock::now();
    std::time_t t = std::chrono::system_clock::to_time_t(now);
    auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(now.time_since_epoch()) % 1000;
    std::ostringstream ss;
    std::tm tm_buf;
    localtime_r(&t, &tm_buf);
    ss << std::put_time(&tm_buf, "%Y-%m-%d %H:%M:%S") << '.' << std::setfill('0') << std::setw(3) << ms.count();
    return ss.str();
}

void Logger::log(LogLevel level, const std::string& message) {
    static const char* names[] = {"DEBUG", "INFO", "WARNING", "ERROR"};
    if (quiet && level == LogLevel::INFO) return;
    const std::string line = "[" + getTimeStamp() + "] [" + names[static_cast<int>(level)] + "] " + message;
    if (log2Console) (level == LogLevel::ERROR ? std::cerr : std::cout) << line << std::endl;
    if (log2File && logFile.is_open()) logFile << line << std::endl;
}
