// A small regular-expression matcher for the patterns a model description uses to name tensors it
// ignores (std::regex drags in locale machinery that clashes with other C++ runtimes in the
// process).  Supported: literals, `.`, `\d \w \s` and escaped punctuation, classes `[a-z_]` and
// `[^...]`, groups `( ... | ... )`, the quantifiers `* + ?`, and the anchors `^ $`.  `search`
// finds the pattern anywhere in the text, as re.search does.
#pragma once

#include <memory>
#include <string>
#include <vector>

namespace sandy {

class Pattern {
public:
    explicit Pattern(const std::string& text);      // throws ValueError on a malformed pattern
    bool search(const std::string& s) const;
    struct Node;
private:
    std::shared_ptr<Node> root_;
};

}  // namespace sandy
