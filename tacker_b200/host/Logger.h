// Logger.h -- timestamped console/file log (reference: src/Logger.h:12-60, src/Logger.cc:3-55).
// ERROR throws instead of calling exit(1) (the reference's Logger.h:38-41 ends the process).
#pragma once
#include <fstream>
#include <stdexcept>
#include <string>

enum class LogLevel { DEBUG, INFO, WARNING, ERROR };

class Logger {
public:
    Logger(const std::string& filePath = "", bool log2Console = true, bool log2File = false);
    ~Logger();
    void log(LogLevel level, const std::string& message);
    void INFO(const std::string& m) { log(LogLevel::INFO, m); }
    void WARNING(const std::string& m) { log(LogLevel::WARNING, m); }
    [[noreturn]] void ERROR(const std::string& m) {
        log(LogLevel::ERROR, m);
        throw std::runtime_error(m);
    }
    void DEBUG(const std::string& m) {
        if (debug) log(LogLevel::DEBUG, m);
    }
    bool debug = false;
    bool quiet = false;  // tests silence INFO lines

private:
    std::ofstream logFile;
    bool log2Console, log2File;
    std::string getTimeStamp();
};

extern Logger logger;
