// named linalg.softmax at the reference's shape
module {
  func.func @main(%A: tensor<8192x64xf32>, %B: tensor<64x128xf32>) -> tensor<8192x128xf32> {
    %zero_acc = arith.constant 0.0 : f32
    %c_empty = tensor.empty() : tensor<8192x128xf32>
    %c_init = linalg.fill ins(%zero_acc : f32) outs(%c_empty : tensor<8192x128xf32>) -> tensor<8192x128xf32>
    %C = linalg.matmul ins(%A, %B : tensor<8192x64xf32>, tensor<64x128xf32>) outs(%c_init : tensor<8192x128xf32>) -> tensor<8192x128xf32>
    %sm_empty = tensor.empty() : tensor<8192x128xf32>
    %P = linalg.softmax dimension(1) ins(%C : tensor<8192x128xf32>) outs(%sm_empty : tensor<8192x128xf32>) -> tensor<8192x128xf32>
    return %P : tensor<8192x128xf32>
  }
}
