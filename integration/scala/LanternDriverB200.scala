package lantern

import scala.virtualization.lms._
import scala.virtualization.lms.common._

/**
  * Drivers for programs staged against liblantern_b200.so.
  *
  * `DslDriverB200` takes the place of `DslDriverCudnn` (DslAPI.scala:995-1016): the same nvcc route, with the
  * library's include and link flags instead of -lcublas -lcudnn.  `LanternDriverB200` takes the place of
  * `LanternDriverCudnn` (DslAPI.scala:1064-1077); it has no kernel maps to splice into the generated file because no
  * kernel is generated: every one lives in the library.
  *
  * LANTERN_B200_HOME names the checkout of the library (the directory that holds include/ and lantern_b200/).
  */
abstract class DslDriverB200[A: Manifest, B: Manifest] extends DslDriverCuda[A, B] { self =>
  override val codegen = new DslGenB200 {
    val IR: self.type = self
  }

  def b200Home: String = sys.env.getOrElse("LANTERN_B200_HOME", ".")

  override def nvccArguments: Seq[String] = Seq(
    "-std=c++17", "-O1", "-lstdc++",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-I", s"$b200Home/include",
    "-L", s"$b200Home/lantern_b200", "-llantern_b200",
    "-Xlinker", s"-rpath=$b200Home/lantern_b200")

  override def eval(a: A) {
    val cudaFileName = s"$dir/$fileName.cu"
    val binaryFileName = s"$dir/$fileName"
    val out = new java.io.PrintWriter(cudaFileName)
    out.println(code)
    out.close()

    new java.io.File(binaryFileName).delete
    import scala.sys.process._
    System.out.println("Compile C++ (lantern_b200) code")
    (s"nvcc $cudaFileName -o $binaryFileName ${nvccArguments.mkString(" ")}": ProcessBuilder).lines.foreach(System.out.println)
    System.out.println("Run C++ (lantern_b200) code")
    (s"$binaryFileName $a": ProcessBuilder).lines.foreach(System.out.println)
  }
}

abstract class LanternDriverB200[A: Manifest, B: Manifest] extends DslDriverB200[A, B]
    with LanternDriver[A, B] with TensorDslB200 with NNModule with Dataset with ONNXLib { self =>
  override def manifestA: Manifest[A] = manifest[A]
  override def manifestB: Manifest[B] = manifest[B]
}
