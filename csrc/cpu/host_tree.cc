// Parser of the algorithm-tree text (grammar in host_tree.h).
#include "host_tree.h"
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <sstream>

namespace hccl {
namespace {

struct Parser {
    const std::string& s;
    size_t i = 0;
    std::string err;
    explicit Parser(const std::string& t) : s(t) {}
    void Ws() { while (i < s.size() && isspace((unsigned char)s[i])) ++i; }
    bool Eat(char c) { Ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return false; }
    std::string Word()
    {
        Ws();
        std::string w;
        while (i < s.size() && (isalnum((unsigned char)s[i]) || s[i] == '_' || s[i] == '-')) w += (char)tolower((unsigned char)s[i++]);
        return w;
    }
    bool Number(double* out)
    {
        Ws();
        char* end = nullptr;
        const double d = strtod(s.c_str() + i, &end);
        if (end == s.c_str() + i || d < 0) return false;
        i = (size_t)(end - s.c_str());
        *out = d;
        return true;
    }
    std::unique_ptr<AlgoTreeNode> Node(int depth)
    {
        if (depth > 8) { err = "tree deeper than 8 levels"; return nullptr; }
        const size_t at = i;
        const std::string w = Word();
        auto n = std::make_unique<AlgoTreeNode>();
        if (w == "seq" || w == "par" || w == "rev") {
            n->kind = w == "seq" ? AlgoTreeNode::Kind::SEQ : w == "par" ? AlgoTreeNode::Kind::PAR : AlgoTreeNode::Kind::REV;
            if (!Eat('(')) { err = "'(' expected after '" + w + "' at column " + std::to_string(i); return nullptr; }
            for (;;) {
                Ws();
                if (n->kind == AlgoTreeNode::Kind::PAR && n->kids.size() == 2 && i < s.size() && (isdigit((unsigned char)s[i]) || s[i] == '.')) {
                    if (!Number(&n->shareA) || !Eat(':') || !Number(&n->shareB) || n->shareA + n->shareB <= 0) { err = "par: shares must read a:b with a + b > 0"; return nullptr; }
                } else {
                    auto k = Node(depth + 1);
                    if (!k) return nullptr;
                    n->kids.push_back(std::move(k));
                }
                if (Eat(',')) continue;
                if (Eat(')')) break;
                err = "',' or ')' expected at column " + std::to_string(i);
                return nullptr;
            }
            const size_t k = n->kids.size();
            if (n->kind == AlgoTreeNode::Kind::SEQ && (k < 2 || k > 3)) { err = "seq takes two or three children"; return nullptr; }
            if (n->kind == AlgoTreeNode::Kind::PAR && k != 2) { err = "par takes two children"; return nullptr; }
            if (n->kind == AlgoTreeNode::Kind::REV && k != 1) { err = "rev takes one child"; return nullptr; }
            if (n->kind == AlgoTreeNode::Kind::SEQ)
                for (size_t c = 0; c + 1 < k; ++c)
                    if (n->kids[c]->kind != AlgoTreeNode::Kind::LEAF) { err = "seq: only the last child may be a subtree"; return nullptr; }
            return n;
        }
        static const char* kLeaves[] = {"mesh", "ring", "nhr", "rhd", "nb"};
        if (std::find(std::begin(kLeaves), std::end(kLeaves), w) == std::end(kLeaves)) {
            err = w.empty() ? "template name expected at column " + std::to_string(at) : "unknown template '" + w + "'";
            return nullptr;
        }
        n->leaf = w;
        return n;
    }
};

}  // namespace

bool ParseAlgoTree(const std::string& text, std::unique_ptr<AlgoTreeNode>* out, std::string* err)
{
    Parser p(text);
    auto n = p.Node(0);
    if (n) {
        p.Ws();
        if (p.i != text.size()) { p.err = "unexpected text at column " + std::to_string(p.i); n.reset(); }
    }
    if (!n) { if (err) *err = p.err; return false; }
    *out = std::move(n);
    return true;
}

std::string AlgoTreeText(const AlgoTreeNode& n)
{
    if (n.kind == AlgoTreeNode::Kind::LEAF) return n.leaf;
    std::ostringstream os;
    os << (n.kind == AlgoTreeNode::Kind::SEQ ? "seq(" : n.kind == AlgoTreeNode::Kind::PAR ? "par(" : "rev(");
    for (size_t i = 0; i < n.kids.size(); ++i) os << (i ? "," : "") << AlgoTreeText(*n.kids[i]);
    if (n.kind == AlgoTreeNode::Kind::PAR && n.shareA + n.shareB > 0) os << "," << n.shareA << ":" << n.shareB;
    os << ")";
    return os.str();
}

uint32_t AlgoTreeQueues(const AlgoTreeNode& n)
{
    if (n.kind == AlgoTreeNode::Kind::LEAF) return 1;
    if (n.kind == AlgoTreeNode::Kind::PAR) return AlgoTreeQueues(*n.kids[0]) + AlgoTreeQueues(*n.kids[1]);
    return AlgoTreeQueues(*n.kids.back());
}

uint32_t AlgoTreeMinLevels(const AlgoTreeNode& n)
{
    switch (n.kind) {
        case AlgoTreeNode::Kind::LEAF: return 1;
        case AlgoTreeNode::Kind::SEQ: return (uint32_t)n.kids.size() - 1 + AlgoTreeMinLevels(*n.kids.back());
        case AlgoTreeNode::Kind::PAR: return std::max(AlgoTreeMinLevels(*n.kids[0]), AlgoTreeMinLevels(*n.kids[1]));
        default: return AlgoTreeMinLevels(*n.kids[0]);
    }
}

}  // namespace hccl
