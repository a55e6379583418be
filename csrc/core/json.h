// Minimal JSON reader (objects, arrays, strings, numbers, true/false/null) for
// rank tables and topology literals.  Values are kept as a small variant tree.
#pragma once
#include <cctype>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace hccl {

struct JsonValue {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JsonValue> arr;
    std::map<std::string, JsonValue> obj;
    const JsonValue* Get(const std::string& k) const
    {
        auto it = obj.find(k);
        return it == obj.end() ? nullptr : &it->second;
    }
    // numbers are often written as strings in rank tables ("rank_id":"0")
    bool AsU64(unsigned long long* out) const
    {
        if (kind == NUM && num >= 0) { *out = (unsigned long long)num; return true; }
        if (kind == STR && !str.empty()) {
            char* end = nullptr;
            unsigned long long v = strtoull(str.c_str(), &end, 10);
            if (*end == 0) { *out = v; return true; }
        }
        return false;
    }
};

class JsonParser {
public:
    explicit JsonParser(const std::string& text) : s_(text) {}
    bool Parse(JsonValue* out, std::string* err)
    {
        pos_ = 0;
        if (!Value(out, 0)) { *err = err_ + " at offset " + std::to_string(pos_); return false; }
        Ws();
        if (pos_ != s_.size()) { *err = "trailing characters at offset " + std::to_string(pos_); return false; }
        return true;
    }

private:
    void Ws()
    {
        for (;;) {
            while (pos_ < s_.size() && isspace((unsigned char)s_[pos_])) ++pos_;
            // rank-table examples carry // comments: skip them
            if (pos_ + 1 < s_.size() && s_[pos_] == '/' && s_[pos_ + 1] == '/') { while (pos_ < s_.size() && s_[pos_] != '\n') ++pos_; continue; }
            break;
        }
    }
    bool Fail(const char* m) { err_ = m; return false; }
    bool Value(JsonValue* v, int depth)
    {
        if (depth > 64) return Fail("nesting too deep");
        Ws();
        if (pos_ >= s_.size()) return Fail("unexpected end");
        char c = s_[pos_];
        if (c == '{') {
            v->kind = JsonValue::OBJ;
            ++pos_;
            Ws();
            if (pos_ < s_.size() && s_[pos_] == '}') { ++pos_; return true; }
            for (;;) {
                Ws();
                JsonValue key;
                if (pos_ >= s_.size() || s_[pos_] != '"' || !String(&key.str)) return Fail("expected a string key");
                Ws();
                if (pos_ >= s_.size() || s_[pos_] != ':') return Fail("expected ':'");
                ++pos_;
                JsonValue val;
                if (!Value(&val, depth + 1)) return false;
                v->obj[key.str] = std::move(val);
                Ws();
                if (pos_ < s_.size() && s_[pos_] == ',') { ++pos_; continue; }
                if (pos_ < s_.size() && s_[pos_] == '}') { ++pos_; return true; }
                return Fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            v->kind = JsonValue::ARR;
            ++pos_;
            Ws();
            if (pos_ < s_.size() && s_[pos_] == ']') { ++pos_; return true; }
            for (;;) {
                JsonValue e;
                if (!Value(&e, depth + 1)) return false;
                v->arr.push_back(std::move(e));
                Ws();
                if (pos_ < s_.size() && s_[pos_] == ',') { ++pos_; continue; }
                if (pos_ < s_.size() && s_[pos_] == ']') { ++pos_; return true; }
                return Fail("expected ',' or ']'");
            }
        }
        if (c == '"') { v->kind = JsonValue::STR; return String(&v->str); }
        if (s_.compare(pos_, 4, "true") == 0) { v->kind = JsonValue::BOOL; v->b = true; pos_ += 4; return true; }
        if (s_.compare(pos_, 5, "false") == 0) { v->kind = JsonValue::BOOL; v->b = false; pos_ += 5; return true; }
        if (s_.compare(pos_, 4, "null") == 0) { v->kind = JsonValue::NUL; pos_ += 4; return true; }
        char* end = nullptr;
        double d = strtod(s_.c_str() + pos_, &end);
        if (end == s_.c_str() + pos_) return Fail("unexpected character");
        v->kind = JsonValue::NUM;
        v->num = d;
        pos_ = (size_t)(end - s_.c_str());
        return true;
    }
    bool String(std::string* out)
    {
        ++pos_;
        out->clear();
        while (pos_ < s_.size() && s_[pos_] != '"') {
            if (s_[pos_] == '\\' && pos_ + 1 < s_.size()) {
                char e = s_[pos_ + 1];
                out->push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e);
                pos_ += 2;
            } else {
                out->push_back(s_[pos_++]);
            }
        }
        if (pos_ >= s_.size()) return Fail("unterminated string");
        ++pos_;
        return true;
    }
    const std::string& s_;
    size_t pos_ = 0;
    std::string err_;
};

}  // namespace hccl
