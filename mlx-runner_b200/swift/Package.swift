// swift-tools-version:5.9
// SwiftPM manifest a host application adds to bind libmlxq (not compiled in this repository: there is no
// Swift toolchain on the build machines; the C header it exposes is exercised from C++ and Python).
import PackageDescription

let package = Package(
    name: "MLXQ",
    products: [.library(name: "MLXQ", targets: ["MLXQ"])],
    targets: [
        // System-library target: the module map re-exports include/mlxq.h and links libmlxq.so.
        .systemLibrary(name: "CMLXQ", path: "Sources/CMLXQ"),
        .target(name: "MLXQ", dependencies: ["CMLXQ"], path: "Sources/MLXQ"),
    ]
)
