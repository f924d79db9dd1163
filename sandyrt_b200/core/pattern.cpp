#include "pattern.h"

#include <functional>

#include "errors.h"

namespace sandy {

struct Pattern::Node {
    enum Kind { Char, Any, Class, Group, Begin, End } kind = Char;
    char ch = 0;
    bool negate = false;
    std::vector<std::pair<char, char>> ranges;                  // Class
    std::vector<std::vector<std::shared_ptr<Node>>> branches;   // Group: alternatives, each a sequence
    int min = 1, max = 1;                                        // repetition; max < 0: unbounded
};

namespace {

using NodePtr = std::shared_ptr<Pattern::Node>;
using Seq = std::vector<NodePtr>;

struct PatternParser {
    const std::string& t;
    size_t pos = 0;
    [[noreturn]] void fail(const std::string& why) const { throw ValueError("bad pattern '" + t + "': " + why); }

    void add_escape(Pattern::Node& n, char c) {
        n.kind = Pattern::Node::Class;
        if (c == 'd') n.ranges = {{'0', '9'}};
        else if (c == 'w') n.ranges = {{'a', 'z'}, {'A', 'Z'}, {'0', '9'}, {'_', '_'}};
        else if (c == 's') n.ranges = {{' ', ' '}, {'\t', '\t'}, {'\n', '\n'}, {'\r', '\r'}};
        else { n.kind = Pattern::Node::Char; n.ch = c; }
    }
    NodePtr atom() {
        auto n = std::make_shared<Pattern::Node>();
        const char c = t[pos++];
        if (c == '.') n->kind = Pattern::Node::Any;
        else if (c == '^') n->kind = Pattern::Node::Begin;
        else if (c == '$') n->kind = Pattern::Node::End;
        else if (c == '\\') {
            if (pos >= t.size()) fail("a lone backslash");
            add_escape(*n, t[pos++]);
        } else if (c == '[') {
            n->kind = Pattern::Node::Class;
            if (pos < t.size() && t[pos] == '^') { n->negate = true; pos++; }
            bool first = true;
            while (true) {
                if (pos >= t.size()) fail("an unterminated class");
                char a = t[pos++];
                if (a == ']' && !first) break;
                first = false;
                if (a == '\\') {
                    if (pos >= t.size()) fail("a lone backslash");
                    Pattern::Node e;
                    add_escape(e, t[pos++]);
                    if (e.kind == Pattern::Node::Class) { n->ranges.insert(n->ranges.end(), e.ranges.begin(), e.ranges.end()); continue; }
                    a = e.ch;
                }
                char b = a;
                if (pos + 1 < t.size() && t[pos] == '-' && t[pos + 1] != ']') { b = t[pos + 1]; pos += 2; }
                n->ranges.emplace_back(a, b);
            }
        } else if (c == '(') {
            n->kind = Pattern::Node::Group;
            if (t.compare(pos, 2, "?:") == 0) pos += 2;
            n->branches = alternatives();
            if (pos >= t.size() || t[pos] != ')') fail("an unterminated group");
            pos++;
        } else if (c == '*' || c == '+' || c == '?') fail("a quantifier with nothing before it");
        else n->ch = c;
        if (pos < t.size() && n->kind != Pattern::Node::Begin && n->kind != Pattern::Node::End) {
            const char q = t[pos];
            if (q == '*') { n->min = 0; n->max = -1; pos++; }
            else if (q == '+') { n->min = 1; n->max = -1; pos++; }
            else if (q == '?') { n->min = 0; n->max = 1; pos++; }
        }
        return n;
    }
    std::vector<Seq> alternatives() {
        std::vector<Seq> out(1);
        while (pos < t.size() && t[pos] != ')') {
            if (t[pos] == '|') { out.emplace_back(); pos++; continue; }
            out.back().push_back(atom());
        }
        return out;
    }
};

using Cont = std::function<bool(size_t)>;

bool match_seq(const Seq& seq, size_t i, const std::string& s, size_t at, const Cont& k);

bool match_once(const Pattern::Node& n, const std::string& s, size_t at, const Cont& k) {
    switch (n.kind) {
        case Pattern::Node::Begin: return at == 0 && k(at);
        case Pattern::Node::End: return at == s.size() && k(at);
        case Pattern::Node::Any: return at < s.size() && s[at] != '\n' && k(at + 1);
        case Pattern::Node::Char: return at < s.size() && s[at] == n.ch && k(at + 1);
        case Pattern::Node::Class: {
            if (at >= s.size()) return false;
            bool in = false;
            for (const auto& r : n.ranges) in = in || (s[at] >= r.first && s[at] <= r.second);
            return in != n.negate && k(at + 1);
        }
        case Pattern::Node::Group:
            for (const Seq& b : n.branches)
                if (match_seq(b, 0, s, at, k)) return true;
            return false;
    }
    return false;
}

bool match_repeat(const Pattern::Node& n, int done, const std::string& s, size_t at, const Cont& k) {
    if (n.max < 0 || done < n.max) {          // greedy: one more first
        const Cont again = [&](size_t next) { return next != at && match_repeat(n, done + 1, s, next, k); };
        if (match_once(n, s, at, again)) return true;
    }
    return done >= n.min && k(at);
}

bool match_seq(const Seq& seq, size_t i, const std::string& s, size_t at, const Cont& k) {
    if (i == seq.size()) return k(at);
    const Pattern::Node& n = *seq[i];
    const Cont rest = [&](size_t next) { return match_seq(seq, i + 1, s, next, k); };
    if (n.min == 1 && n.max == 1) return match_once(n, s, at, rest);
    return match_repeat(n, 0, s, at, rest);
}

}  // namespace

Pattern::Pattern(const std::string& text) {
    PatternParser p{text};
    root_ = std::make_shared<Node>();
    root_->kind = Node::Group;
    root_->branches = p.alternatives();
    if (p.pos != text.size()) p.fail("an unmatched ')'");
}

bool Pattern::search(const std::string& s) const {
    const Cont done = [](size_t) { return true; };
    for (size_t start = 0; start <= s.size(); start++)
        if (match_once(*root_, s, start, done)) return true;
    return false;
}

}  // namespace sandy
