// named linalg.softmax at the reference's shape
!t0 = tensor<8192x64xf32>
!t1 = tensor<64x128xf32>
!t2 = tensor<8192x128xf32>
module {
  func.func @main(%A: !t0, %B: !t1) -> !t2 {
    %zero_acc = arith.constant 0.0 : f32
    %c_empty = tensor.empty() : !t2
    %c_init = linalg.fill ins(%zero_acc : f32) outs(%c_empty : !t2) -> !t2
    %C = linalg.matmul ins(%A, %B : !t0, !t1) outs(%c_init : !t2) -> !t2
    %sm_empty = tensor.empty() : !t2
    %P = linalg.softmax dimension(1) ins(%C : !t2) outs(%sm_empty : !t2) -> !t2
    return %P : !t2
  }
}
