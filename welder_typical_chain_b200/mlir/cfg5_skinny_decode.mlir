// configuration 5: X[16,4096] . W[4096,32000], f16 probabilities
#m0 = affine_map<(d0, d1) -> (d0, d1)>
#m1 = affine_map<(d0, d1) -> (d0)>
!t0 = tensor<16x4096xf16>
!t1 = tensor<4096x32000xf16>
!t2 = tensor<16x32000xf16>
!t3 = tensor<16x32000xf32>
!t4 = tensor<16xf32>
module {
  func.func @main(%A: !t0, %B: !t1) -> !t2 {
    %zero_acc = arith.constant 0.0 : f32
    %c_empty = tensor.empty() : !t3
    %c_init = linalg.fill ins(%zero_acc : f32) outs(%c_empty : !t3) -> !t3
    %C = linalg.matmul ins(%A, %B : !t0, !t1) outs(%c_init : !t3) -> !t3
    %neg_inf = arith.constant -3.4028235e+38 : f32
    %zero = arith.constant 0.0 : f32
    // row maximum
    %max_empty = tensor.empty() : !t4
    %max_init = linalg.fill ins(%neg_inf : f32) outs(%max_empty : !t4) -> !t4
    %max = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%C : !t3) outs(%max_init : !t4) {
      ^bb0(%in: f32, %acc: f32):
        %m = arith.maximumf %in, %acc : f32
        linalg.yield %m : f32
      } -> !t4
    // exp(x - max)
    %exp_empty = tensor.empty() : !t3
    %exp = linalg.generic {indexing_maps = [#m0, #m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%C, %max : !t3, !t4) outs(%exp_empty : !t3) {
      ^bb0(%x: f32, %m: f32, %o: f32):
        %d = arith.subf %x, %m : f32
        %e = math.exp %d : f32
        linalg.yield %e : f32
      } -> !t3
    // row sum
    %sum_empty = tensor.empty() : !t4
    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : !t4) -> !t4
    %sum = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%exp : !t3) outs(%sum_init : !t4) {
      ^bb0(%in: f32, %acc: f32):
        %s = arith.addf %in, %acc : f32
        linalg.yield %s : f32
      } -> !t4
    // normalise
    %div_empty = tensor.empty() : !t3
    %P = linalg.generic {indexing_maps = [#m0, #m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%exp, %sum : !t3, !t4) outs(%div_empty : !t3) {
      ^bb0(%e: f32, %s: f32, %o: f32):
        %q = arith.divf %e, %s : f32
        linalg.yield %q : f32
      } -> !t3
    // probabilities in the output type
    %P16_empty = tensor.empty() : !t2
    %P16 = linalg.generic {indexing_maps = [#m0, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%P : !t3) outs(%P16_empty : !t2) {
      ^bb0(%x: f32, %o: f16):
        %y = arith.truncf %x : f32 to f16
        linalg.yield %y : f16
      } -> !t2
    return %P16 : !t2
  }
}
