// row variance of A[32,256]: sum -> mean -> squared differences -> sum -> variance -> broadcast
#m0 = affine_map<(d0, d1) -> (d0, d1)>
#m1 = affine_map<(d0, d1) -> (d0)>
#m2 = affine_map<(d0) -> (d0)>
!t0 = tensor<32x256xf32>
!t1 = tensor<32xf32>
module {
  func.func @main(%A: !t0) -> !t0 {
    %zero = arith.constant 0.0 : f32
    // row sum -> mean
    %sum_empty = tensor.empty() : !t1
    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : !t1) -> !t1
    %sum = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%A : !t0) outs(%sum_init : !t1) {
      ^bb0(%in: f32, %acc: f32):
        %r = arith.addf %in, %acc : f32
        linalg.yield %r : f32
      } -> !t1
    %mean_empty = tensor.empty() : !t1
    %mean = linalg.generic {indexing_maps = [#m2, #m2], iterator_types = ["parallel"]}
        ins(%sum : !t1) outs(%mean_empty : !t1) {
      ^bb0(%in: f32, %o: f32):
        %inv = arith.constant 0.00390625 : f32
        %v = arith.mulf %in, %inv : f32
        linalg.yield %v : f32
      } -> !t1
    // (a - mean)^2
    %sq_empty = tensor.empty() : !t0
    %sq = linalg.generic {indexing_maps = [#m0, #m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%A, %mean : !t0, !t1) outs(%sq_empty : !t0) {
      ^bb0(%a: f32, %m: f32, %o: f32):
        %d = arith.subf %a, %m : f32
        %s = arith.mulf %d, %d : f32
        linalg.yield %s : f32
      } -> !t0
    // row sum of the squares -> variance
    %sumsq_empty = tensor.empty() : !t1
    %sumsq_init = linalg.fill ins(%zero : f32) outs(%sumsq_empty : !t1) -> !t1
    %sumsq = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%sq : !t0) outs(%sumsq_init : !t1) {
      ^bb0(%in: f32, %acc: f32):
        %r = arith.addf %in, %acc : f32
        linalg.yield %r : f32
      } -> !t1
    %var_empty = tensor.empty() : !t1
    %var = linalg.generic {indexing_maps = [#m2, #m2], iterator_types = ["parallel"]}
        ins(%sumsq : !t1) outs(%var_empty : !t1) {
      ^bb0(%in: f32, %o: f32):
        %inv = arith.constant 0.00390625 : f32
        %v = arith.mulf %in, %inv : f32
        linalg.yield %v : f32
      } -> !t1
    // broadcast along the row
    %out_empty = tensor.empty() : !t0
    %out = linalg.generic {indexing_maps = [#m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%var : !t1) outs(%out_empty : !t0) {
      ^bb0(%v: f32, %o: f32):
        linalg.yield %v : f32
      } -> !t0
    return %out : !t0
  }
}
