// row softmax of X[32,256] (max -> exp -> sum -> divide), no matmul
#m0 = affine_map<(d0, d1) -> (d0, d1)>
#m1 = affine_map<(d0, d1) -> (d0)>
!t0 = tensor<32x256xf32>
!t1 = tensor<32xf32>
module {
  func.func @main(%X: !t0) -> !t0 {
    %neg_inf = arith.constant -3.4028235e+38 : f32
    %zero = arith.constant 0.0 : f32
    // row maximum
    %max_empty = tensor.empty() : !t1
    %max_init = linalg.fill ins(%neg_inf : f32) outs(%max_empty : !t1) -> !t1
    %max = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%X : !t0) outs(%max_init : !t1) {
      ^bb0(%in: f32, %acc: f32):
        %m = arith.maximumf %in, %acc : f32
        linalg.yield %m : f32
      } -> !t1
    // exp(x - max)
    %exp_empty = tensor.empty() : !t0
    %exp = linalg.generic {indexing_maps = [#m0, #m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%X, %max : !t0, !t1) outs(%exp_empty : !t0) {
      ^bb0(%x: f32, %m: f32, %o: f32):
        %d = arith.subf %x, %m : f32
        %e = math.exp %d : f32
        linalg.yield %e : f32
      } -> !t0
    // row sum
    %sum_empty = tensor.empty() : !t1
    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : !t1) -> !t1
    %sum = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%exp : !t0) outs(%sum_init : !t1) {
      ^bb0(%in: f32, %acc: f32):
        %s = arith.addf %in, %acc : f32
        linalg.yield %s : f32
      } -> !t1
    // normalise
    %div_empty = tensor.empty() : !t0
    %P = linalg.generic {indexing_maps = [#m0, #m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%exp, %sum : !t0, !t1) outs(%div_empty : !t0) {
      ^bb0(%e: f32, %s: f32, %o: f32):
        %q = arith.divf %e, %s : f32
        linalg.yield %q : f32
      } -> !t0
    return %P : !t0
  }
}
