// Small text helpers shared by the input readers (host only).
#pragma once

#include <algorithm>
#include <cctype>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace dsmd::host {

inline std::string trimmed(const std::string& s, const char* blanks = " \t\r\n") {
    const size_t a = s.find_first_not_of(blanks);
    if (a == std::string::npos) return std::string();
    const size_t b = s.find_last_not_of(blanks);
    return s.substr(a, b - a + 1);
}

inline std::string lowered(std::string s) {
    for (char& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    return s;
}

inline std::string uppered(std::string s) {
    for (char& c : s) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
    return s;
}

// A file name as it may appear in an input: blanks trimmed, one pair of enclosing double quotes removed.
inline std::string clean_file_name(const std::string& raw) {
    std::string s = trimmed(raw);
    if (s.size() >= 2 && s.front() == '"' && s.back() == '"') s = s.substr(1, s.size() - 2);
    return s;
}

inline std::vector<std::string> words(const std::string& line) {
    std::istringstream in(line);
    std::vector<std::string> out;
    std::string w;
    while (in >> w) out.push_back(w);
    return out;
}

inline std::vector<std::string> comma_list(const std::string& text) {
    std::vector<std::string> out;
    std::stringstream in(text);
    std::string item;
    while (std::getline(in, item, ',')) {
        item = trimmed(item);
        if (!item.empty()) out.push_back(item);
    }
    return out;
}

// std::stod / std::stoi semantics (leading number accepted, trailing text ignored) with a message that names the key.
inline double number_of(const std::string& key, const std::string& value) {
    try {
        return std::stod(value);
    } catch (const std::exception&) {
        throw std::runtime_error("cannot read a number for '" + key + "' from '" + value + "'");
    }
}

inline long long integer_of(const std::string& key, const std::string& value) {
    try {
        return std::stoll(value);
    } catch (const std::exception&) {
        throw std::runtime_error("cannot read an integer for '" + key + "' from '" + value + "'");
    }
}

}  // namespace dsmd::host
