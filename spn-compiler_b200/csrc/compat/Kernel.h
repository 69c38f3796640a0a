// spnc::Kernel -- the value a compilation returns and an execution takes.
// Same constructor, accessors and enumerators as the reference's common/include/Kernel.h:20-126, so that
// code written against it compiles unchanged; here fileName() names a spnb plan file.
#pragma once
#include <cstddef>
#include <functional>
#include <string>

namespace spnc {

enum KernelQueryType : unsigned { JOINT_QUERY = 1 };
enum KernelTarget : unsigned { CPU = 1, CUDA = 2 };

class Kernel {
 public:
  Kernel(const std::string& fileName, const std::string& kernelName, unsigned queryType, unsigned target,
         unsigned batchSize, unsigned numFeatures, unsigned bytesPerFeature, unsigned numResults,
         unsigned bytesPerResult, const std::string& dataType)
      : file_(fileName), name_(kernelName), id_(std::hash<std::string>{}(fileName + kernelName)), query_(queryType),
        target_(target), batch_(batchSize), features_(numFeatures), featureBytes_(bytesPerFeature),
        results_(numResults), resultBytes_(bytesPerResult), dtype_(dataType) {}

  std::string fileName() const { return file_; }
  const std::string& kernelName() const { return name_; }
  size_t unique_id() const { return id_; }
  unsigned queryType() const { return query_; }
  unsigned target() const { return target_; }
  unsigned batchSize() const { return batch_; }
  unsigned numFeatures() const { return features_; }
  unsigned bytesPerFeature() const { return featureBytes_; }
  unsigned numResults() const { return results_; }
  unsigned bytesPerResult() const { return resultBytes_; }
  const std::string& dataType() const { return dtype_; }

 private:
  std::string file_, name_;
  size_t id_;
  unsigned query_, target_, batch_, features_, featureBytes_, results_, resultBytes_;
  std::string dtype_;
};

}  // namespace spnc
