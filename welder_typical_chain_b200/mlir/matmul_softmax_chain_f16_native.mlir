// f16 operands, f16 matmul result, f32 softmax, f32 result
#m0 = affine_map<(d0, d1) -> (d0, d1)>
#m1 = affine_map<(d0, d1) -> (d0)>
!t0 = tensor<8192x64xf16>
!t1 = tensor<64x128xf16>
!t2 = tensor<8192x128xf32>
!t3 = tensor<8192x128xf16>
!t4 = tensor<8192xf32>
module {
  func.func @main(%A: !t0, %B: !t1) -> !t2 {
    %zero_acc = arith.constant 0.0 : f16
    %c_empty = tensor.empty() : !t3
    %c_init = linalg.fill ins(%zero_acc : f16) outs(%c_empty : !t3) -> !t3
    %C = linalg.matmul ins(%A, %B : !t0, !t1) outs(%c_init : !t3) -> !t3
    // widen the matmul result before the softmax
    %C32_empty = tensor.empty() : !t2
    %C32 = linalg.generic {indexing_maps = [#m0, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%C : !t3) outs(%C32_empty : !t2) {
      ^bb0(%x: f16, %o: f32):
        %y = arith.extf %x : f16 to f32
        linalg.yield %y : f32
      } -> !t2
    %neg_inf = arith.constant -3.4028235e+38 : f32
    %zero = arith.constant 0.0 : f32
    // row maximum
    %max_empty = tensor.empty() : !t4
    %max_init = linalg.fill ins(%neg_inf : f32) outs(%max_empty : !t4) -> !t4
    %max = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%C32 : !t2) outs(%max_init : !t4) {
      ^bb0(%in: f32, %acc: f32):
        %m = arith.maximumf %in, %acc : f32
        linalg.yield %m : f32
      } -> !t4
    // exp(x - max)
    %exp_empty = tensor.empty() : !t2
    %exp = linalg.generic {indexing_maps = [#m0, #m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%C32, %max : !t2, !t4) outs(%exp_empty : !t2) {
      ^bb0(%x: f32, %m: f32, %o: f32):
        %d = arith.subf %x, %m : f32
        %e = math.exp %d : f32
        linalg.yield %e : f32
      } -> !t2
    // row sum
    %sum_empty = tensor.empty() : !t4
    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : !t4) -> !t4
    %sum = linalg.generic {indexing_maps = [#m0, #m1], iterator_types = ["parallel", "reduction"]}
        ins(%exp : !t2) outs(%sum_init : !t4) {
      ^bb0(%in: f32, %acc: f32):
        %s = arith.addf %in, %acc : f32
        linalg.yield %s : f32
      } -> !t4
    // normalise
    %div_empty = tensor.empty() : !t2
    %P = linalg.generic {indexing_maps = [#m0, #m1, #m0], iterator_types = ["parallel", "parallel"]}
        ins(%exp, %sum : !t2, !t4) outs(%div_empty : !t2) {
      ^bb0(%e: f32, %s: f32, %o: f32):
        %q = arith.divf %e, %s : f32
        linalg.yield %q : f32
      } -> !t2
    return %P : !t2
  }
}
