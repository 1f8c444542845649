// configuration 3: 64 x (Q[2048,128] . Kt[128,2048]), named softmax, f16 probabilities
#m0 = affine_map<(d0, d1, d2) -> (d0, d1, d2)>
!t0 = tensor<64x2048x128xf16>
!t1 = tensor<64x128x2048xf16>
!t2 = tensor<64x2048x2048xf16>
!t3 = tensor<64x2048x2048xf32>
module {
  func.func @main(%A: !t0, %B: !t1) -> !t2 {
    %zero_acc = arith.constant 0.0 : f32
    %c_empty = tensor.empty() : !t3
    %c_init = linalg.fill ins(%zero_acc : f32) outs(%c_empty : !t3) -> !t3
    %C = linalg.batch_matmul ins(%A, %B : !t0, !t1) outs(%c_init : !t3) -> !t3
    %scale = arith.constant 0.08838834764831845 : f32
    // scaled logits
    %V_empty = tensor.empty() : !t3
    %V = linalg.generic {indexing_maps = [#m0, #m0], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%C : !t3) outs(%V_empty : !t3) {
      ^bb0(%x: f32, %o: f32):
        %y = arith.mulf %x, %scale : f32
        linalg.yield %y : f32
      } -> !t3
    %sm_empty = tensor.empty() : !t3
    %P = linalg.softmax dimension(2) ins(%V : !t3) outs(%sm_empty : !t3) -> !t3
    // probabilities in the output type
    %P16_empty = tensor.empty() : !t2
    %P16 = linalg.generic {indexing_maps = [#m0, #m0], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%P : !t3) outs(%P16_empty : !t2) {
      ^bb0(%x: f32, %o: f16):
        %y = arith.truncf %x : f32 to f16
        linalg.yield %y : f16
      } -> !t2
    return %P16 : !t2
  }
}
