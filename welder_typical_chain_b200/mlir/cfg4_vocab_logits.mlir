// configuration 4: hidden[8192,4096] . W[4096,32000], f16 probabilities
module {
  func.func @main(%A: tensor<8192x4096xf16>, %B: tensor<4096x32000xf16>) -> tensor<8192x32000xf16> {
    %zero_acc = arith.constant 0.0 : f32
    %c_empty = tensor.empty() : tensor<8192x32000xf32>
    %c_init = linalg.fill ins(%zero_acc : f32) outs(%c_empty : tensor<8192x32000xf32>) -> tensor<8192x32000xf32>
    %C = linalg.matmul ins(%A, %B : tensor<8192x4096xf16>, tensor<4096x32000xf16>) outs(%c_init : tensor<8192x32000xf32>) -> tensor<8192x32000xf32>
    %neg_inf = arith.constant -3.4028235e+38 : f32
    %zero = arith.constant 0.0 : f32
    // row maximum
    %max_empty = tensor.empty() : tensor<8192xf32>
    %max_init = linalg.fill ins(%neg_inf : f32) outs(%max_empty : tensor<8192xf32>) -> tensor<8192xf32>
    %max = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]}
        ins(%C : tensor<8192x32000xf32>) outs(%max_init : tensor<8192xf32>) {
      ^bb0(%in: f32, %acc: f32):
        %m = arith.maximumf %in, %acc : f32
        linalg.yield %m : f32
      } -> tensor<8192xf32>
    // exp(x - max)
    %exp_empty = tensor.empty() : tensor<8192x32000xf32>
    %exp = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%C, %max : tensor<8192x32000xf32>, tensor<8192xf32>) outs(%exp_empty : tensor<8192x32000xf32>) {
      ^bb0(%x: f32, %m: f32, %o: f32):
        %d = arith.subf %x, %m : f32
        %e = math.exp %d : f32
        linalg.yield %e : f32
      } -> tensor<8192x32000xf32>
    // row sum
    %sum_empty = tensor.empty() : tensor<8192xf32>
    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : tensor<8192xf32>) -> tensor<8192xf32>
    %sum = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]}
        ins(%exp : tensor<8192x32000xf32>) outs(%sum_init : tensor<8192xf32>) {
      ^bb0(%in: f32, %acc: f32):
        %s = arith.addf %in, %acc : f32
        linalg.yield %s : f32
      } -> tensor<8192xf32>
    // normalise
    %div_empty = tensor.empty() : tensor<8192x32000xf32>
    %P = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%exp, %sum : tensor<8192x32000xf32>, tensor<8192xf32>) outs(%div_empty : tensor<8192x32000xf32>) {
      ^bb0(%e: f32, %s: f32, %o: f32):
        %q = arith.divf %e, %s : f32
        linalg.yield %q : f32
      } -> tensor<8192x32000xf32>
    // probabilities in the output type
    %P16_empty = tensor.empty() : tensor<8192x32000xf16>
    %P16 = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"]}
        ins(%P : tensor<8192x32000xf32>) outs(%P16_empty : tensor<8192x32000xf16>) {
      ^bb0(%x: f32, %o: f16):
        %y = arith.truncf %x : f32 to f16
        linalg.yield %y : f16
      } -> tensor<8192x32000xf16>
    return %P16 : tensor<8192x32000xf16>
  }
}
