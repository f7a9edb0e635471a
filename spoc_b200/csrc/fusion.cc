// fusion.cc — placeholder, replaced below
#include "ir.hpp"
#include "../../include/sb200.h"
namespace sb200 {
int ir_can_fuse(const std::string&, const std::string&, const std::string&, bool*, std::string* err) { *err = "not implemented"; return SB200_ERR_UNSUPPORTED; }
int ir_fuse(const std::string&, const std::string&, const std::string&, std::string*, std::string* err) { *err = "not implemented"; return SB200_ERR_UNSUPPORTED; }
int ir_fuse_pipeline(const std::vector<std::string>&, std::string*, std::vector<std::string>*, std::string* err) { *err = "not implemented"; return SB200_ERR_UNSUPPORTED; }
}
