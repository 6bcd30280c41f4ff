// swift-tools-version:6.0
// NOT COMPILED HERE: this repository's image has no swift toolchain.  The two targets below are what the
// reference's Package.swift gains to call libleviathan_cuda.so; LeviathanCore would list "LeviathanCUDA" in
// its dependencies and select the backend where it selects Q4MetalBackend today.
import PackageDescription

let package = Package(
    name: "leviathan-cuda",
    targets: [
        .systemLibrary(
            name: "CLeviathanCUDA",
            path: "Sources/CLeviathanCUDA"
        ),
        .target(
            name: "LeviathanCUDA",
            dependencies: ["CLeviathanCUDA"],
            path: "Sources/LeviathanCUDA"
        ),
    ]
)
