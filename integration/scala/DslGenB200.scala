package lantern

import scala.virtualization.lms._
import scala.virtualization.lms.common._

/**
  * Code generator for programs staged against `BackendB200` (TensorDslB200.scala).
  *
  * Takes the place of `DslGenCublas` / `DslGenCudnn` (DslAPI.scala:425-900).  Those traits print a runtime into
  * every generated file: the CUDA_CALL / CUBLAS_CALL / CUDNN_CALL macros, the bump arena (`gpuMallocBase`,
  * `myGpuMalloc`, `myGpuFree`) and about forty-five `__global__` kernels.  Here all of that lives in
  * liblantern_b200.so, so the generated file only needs the header, one error macro and a link flag.
  *
  * The nodes of `GPUOps` (common/GPUOps.scala: `NewGPUArray`, `gpu_array_copy_*`) keep working unchanged: the two
  * strings `CudaGenGPUOps` builds for them are overridden to name the library's arena and its stream-ordered copies.
  * That matters for correctness, not only for tidiness: the library issues its kernels on its own non-blocking
  * stream, and a plain `cudaMemcpy` on the legacy default stream is not ordered against that stream.
  */
trait DslGenB200 extends DslGenBase with CudaGenGPUOps {
  val IR: DslGPUExp
  import IR._

  override def templateHeaders: Seq[String] =
    super.templateHeaders ++ Seq("<initializer_list>", "<cuda_runtime.h>", "\"lantern_b200.h\"")

  // Print-and-exit on error, the convention of CUDA_CALL (DslAPI.scala:435-451).  The library itself already exits in
  // its default (fatal) mode; the macro also covers a host that switched it off with ltb_set_fatal(0).
  override def templateRawCode: String = super.templateRawCode +
    """
      |#define LTB_CALL(f) { \
      |  int ltb_status_ = (f); \
      |  if (ltb_status_ != 0) { \
      |    char ltb_msg_[512]; ltb_last_error(ltb_msg_, 512); \
      |    fprintf(stderr, "lantern_b200 error %d at %s:%d: %s\n", ltb_status_, __FILE__, __LINE__, ltb_msg_); \
      |    exit(-ltb_status_); \
      |  } \
      |}
      |#ifndef HEAP_SIZE
      |#define HEAP_SIZE 8589934608  // 8 GiB + 16, the reference's arena (DslAPI.scala:453)
      |#endif
      |""".stripMargin

  // NewGPUArray(n): the library's arena, zero at hand-out like myGpuMalloc over a memset arena (DslAPI.scala:453-473).
  override def getCudaMallocArenaString(count: String, dataType: String): String =
    "(" + dataType + "*)ltb_malloc((size_t)(" + count + ") * sizeof(" + dataType + "))"

  // gpu_array_copy_*: ordered on the library's stream; the device-to-host form blocks, as cudaMemcpy does.
  override def cudaMemcpy(dest: String, src: String, count: String, dataType: String, direction: CopyDirection.Value): String = {
    val fn = direction match {
      case CopyDirection.HostToDevice => "ltb_h2d"
      case CopyDirection.DeviceToHost => "ltb_d2h"
      case CopyDirection.DeviceToDevice => "ltb_d2d"
    }
    s"LTB_CALL($fn($dest, $src, (size_t)($count) * sizeof($dataType)));"
  }
}
