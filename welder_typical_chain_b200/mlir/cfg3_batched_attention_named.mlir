// configuration 3: 64 x (Q[2048,128] . Kt[128,2048]), named softmax, f16 probabilities
module {
  func.func @main(%A: tensor<64x2048x128xf16>, %B: tensor<64x128x2048xf16>) -> tensor<64x2048x2048xf16> {
    %zero_acc = arith.constant 0.0 : f32
    %c_empty = tensor.empty() : tensor<64x2048x2048xf32>
    %c_init = linalg.fill ins(%zero_acc : f32) outs(%c_empty : tensor<64x2048x2048xf32>) -> tensor<64x2048x2048xf32>
    %C = linalg.batch_matmul ins(%A, %B : tensor<64x2048x128xf16>, tensor<64x128x2048xf16>) outs(%c_init : tensor<64x2048x2048xf32>) -> tensor<64x2048x2048xf32>
    %scale = arith.constant 0.08838834764831845 : f32
    // scaled logits
    %V_empty = tensor.empty() : tensor<64x2048x2048xf32>
    %V = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d1, d2)>, affine_map<(d0, d1, d2) -> (d0, d1, d2)>], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%C : tensor<64x2048x2048xf32>) outs(%V_empty : tensor<64x2048x2048xf32>) {
      ^bb0(%x: f32, %o: f32):
        %y = arith.mulf %x, %scale : f32
        linalg.yield %y : f32
      } -> tensor<64x2048x2048xf32>
    %sm_empty = tensor.empty() : tensor<64x2048x2048xf32>
    %P = linalg.softmax dimension(2) ins(%V : tensor<64x2048x2048xf32>) outs(%sm_empty : tensor<64x2048x2048xf32>) -> tensor<64x2048x2048xf32>
    // probabilities in the output type
    %P16_empty = tensor.empty() : tensor<64x2048x2048xf16>
    %P16 = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d1, d2)>, affine_map<(d0, d1, d2) -> (d0, d1, d2)>], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%P : tensor<64x2048x2048xf32>) outs(%P16_empty : tensor<64x2048x2048xf16>) {
      ^bb0(%x: f32, %o: f16):
        %y = arith.truncf %x : f32 to f16
        linalg.yield %y : f16
      } -> tensor<64x2048x2048xf16>
    return %P16 : tensor<64x2048x2048xf16>
  }
}
