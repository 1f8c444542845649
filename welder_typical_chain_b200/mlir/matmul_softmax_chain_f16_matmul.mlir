// f32 arguments rounded to f16, f16 matmul result, f32 softmax, f32 result
module {
  func.func @main(%A: tensor<8192x64xf32>, %B: tensor<64x128xf32>) -> tensor<8192x128xf32> {
    // A rounded to f16 for the matmul
    %An_empty = tensor.empty() : tensor<8192x64xf16>
    %An = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%A : tensor<8192x64xf32>) outs(%An_empty : tensor<8192x64xf16>) {
      ^bb0(%x: f32, %o: f16):
        %y = arith.truncf %x : f32 to f16
        linalg.yield %y : f16
      } -> tensor<8192x64xf16>
    // B rounded to f16 for the matmul
    %Bn_empty = tensor.empty() : tensor<64x128xf16>
    %Bn = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%B : tensor<64x128xf32>) outs(%Bn_empty : tensor<64x128xf16>) {
      ^bb0(%x: f32, %o: f16):
        %y = arith.truncf %x : f32 to f16
        linalg.yield %y : f16
      } -> tensor<64x128xf16>
    %zero_acc = arith.constant 0.0 : f16
    %c_empty = tensor.empty() : tensor<8192x128xf16>
    %c_init = linalg.fill ins(%zero_acc : f16) outs(%c_empty : tensor<8192x128xf16>) -> tensor<8192x128xf16>
    %C = linalg.matmul ins(%An, %Bn : tensor<8192x64xf16>, tensor<64x128xf16>) outs(%c_init : tensor<8192x128xf16>) -> tensor<8192x128xf16>
    // widen the matmul result before the softmax
    %C32_empty = tensor.empty() : tensor<8192x128xf32>
    %C32 = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%C : tensor<8192x128xf16>) outs(%C32_empty : tensor<8192x128xf32>) {
      ^bb0(%x: f16, %o: f32):
        %y = arith.extf %x : f16 to f32
        linalg.yield %y : f32
      } -> tensor<8192x128xf32>
    %neg_inf = arith.constant -3.4028235e+38 : f32
    %zero = arith.constant 0.0 : f32
    // row maximum
    %max_empty = tensor.empty() : tensor<8192xf32>
    %max_init = linalg.fill ins(%neg_inf : f32) outs(%max_empty : tensor<8192xf32>) -> tensor<8192xf32>
    %max = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]}
        ins(%C32 : tensor<8192x128xf32>) outs(%max_init : tensor<8192xf32>) {
      ^bb0(%in: f32, %acc: f32):
        %m = arith.maximumf %in, %acc : f32
        linalg.yield %m : f32
      } -> tensor<8192xf32>
    // exp(x - max)
    %exp_empty = tensor.empty() : tensor<8192x128xf32>
    %exp = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%C32, %max : tensor<8192x128xf32>, tensor<8192xf32>) outs(%exp_empty : tensor<8192x128xf32>) {
      ^bb0(%x: f32, %m: f32, %o: f32):
        %d = arith.subf %x, %m : f32
        %e = math.exp %d : f32
        linalg.yield %e : f32
      } -> tensor<8192x128xf32>
    // row sum
    %sum_empty = tensor.empty() : tensor<8192xf32>
    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : tensor<8192xf32>) -> tensor<8192xf32>
    %sum = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]}
        ins(%exp : tensor<8192x128xf32>) outs(%sum_init : tensor<8192xf32>) {
      ^bb0(%in: f32, %acc: f32):
        %s = arith.addf %in, %acc : f32
        linalg.yield %s : f32
      } -> tensor<8192xf32>
    // normalise
    %div_empty = tensor.empty() : tensor<8192x128xf32>
    %P = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%exp, %sum : tensor<8192x128xf32>, tensor<8192xf32>) outs(%div_empty : tensor<8192x128xf32>) {
      ^bb0(%e: f32, %s: f32, %o: f32):
        %q = arith.divf %e, %s : f32
        linalg.yield %q : f32
      } -> tensor<8192x128xf32>
    return %P : tensor<8192x128xf32>
  }
}
