// TEST INFRASTRUCTURE, not product code.
//
// Link stub for the reference build in this folder's Makefile.  The reference's
// src/core/source/manager.cpp asks a GIR graph for two debug strings
// (include/camel/compile/gir/graph.h:210-211) that are only used to decorate error-site
// text.  The graph compiler is not part of the tensor path and is not built here, so the two
// accessors are given empty bodies.
#include "camel/compile/gir/graph.h"

#include <string>

namespace camel::compile::gir {
static const std::string kEmpty;
const std::string &Graph::nodeDebugEntityId(const Node *) const { return kEmpty; }
const std::string &Graph::nodePortName(const Node *) const { return kEmpty; }
} // namespace camel::compile::gir
