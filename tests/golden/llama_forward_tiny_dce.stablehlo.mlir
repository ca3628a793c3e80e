module @jit_sfn attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<8xf32>, %arg1: tensor<2x8xf32>, %arg2: tensor<2x8xf32>, %arg3: tensor<8xf32>, %arg4: tensor<2x16x8xf32>, %arg5: tensor<2x8x16xf32>, %arg6: tensor<2x16x8xf32>, %arg7: tensor<2x8x8xf32>, %arg8: tensor<2x8x8xf32>, %arg9: tensor<2x8x8xf32>, %arg10: tensor<2x8x8xf32>, %arg11: tensor<2x2x8xf32>, %arg12: tensor<2x2x8xf32>) -> (tensor<8xf32> {jax.result_info = ""}) {
    %0 = stablehlo.slice %arg1 [0:1, 0:8] : (tensor<2x8xf32>) -> tensor<1x8xf32>
    %1 = stablehlo.reshape %0 : (tensor<1x8xf32>) -> tensor<8xf32>
    %2 = stablehlo.dot_general %arg0, %arg0, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8xf32>, tensor<8xf32>) -> tensor<f32>
    %cst = stablehlo.constant dense<8.000000e+00> : tensor<f32>
    %3 = stablehlo.divide %2, %cst : tensor<f32>
    %cst_0 = stablehlo.constant dense<1.000000e-05> : tensor<f32>
    %4 = stablehlo.add %3, %cst_0 : tensor<f32>
    %5 = stablehlo.sqrt %4 : tensor<f32>
    %cst_1 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %6 = stablehlo.divide %cst_1, %5 : tensor<f32>
    %7 = stablehlo.multiply %1, %arg0 : tensor<8xf32>
    %8 = stablehlo.broadcast_in_dim %6, dims = [] : (tensor<f32>) -> tensor<8xf32>
    %9 = stablehlo.multiply %7, %8 : tensor<8xf32>
    %10 = stablehlo.slice %arg9 [0:1, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %11 = stablehlo.reshape %10 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %12 = stablehlo.dot_general %11, %9, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %13 = stablehlo.slice %arg7 [0:1, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %14 = stablehlo.reshape %13 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %15 = stablehlo.dot_general %14, %9, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %16 = stablehlo.slice %arg10 [0:1, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %17 = stablehlo.reshape %16 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %18 = stablehlo.dot_general %17, %9, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %19 = stablehlo.reshape %12 : (tensor<8xf32>) -> tensor<4x2xf32>
    %20 = stablehlo.reshape %15 : (tensor<8xf32>) -> tensor<4x2xf32>
    %cst_2 = stablehlo.constant dense<[[[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]], [[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]]]> : tensor<4x2x2xf32>
    %21 = stablehlo.dot_general %cst_2, %20, batching_dims = [0] x [0], contracting_dims = [2] x [1], precision = [DEFAULT, DEFAULT] : (tensor<4x2x2xf32>, tensor<4x2xf32>) -> tensor<4x2xf32>
    %22 = stablehlo.reshape %21 : (tensor<4x2xf32>) -> tensor<8xf32>
    %cst_3 = stablehlo.constant dense<[[[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]], [[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]]]> : tensor<4x2x2xf32>
    %23 = stablehlo.dot_general %cst_3, %19, batching_dims = [0] x [0], contracting_dims = [2] x [1], precision = [DEFAULT, DEFAULT] : (tensor<4x2x2xf32>, tensor<4x2xf32>) -> tensor<4x2xf32>
    %24 = stablehlo.reshape %23 : (tensor<4x2xf32>) -> tensor<8xf32>
    %25 = stablehlo.slice %arg11 [0:1, 0:2, 0:8] : (tensor<2x2x8xf32>) -> tensor<1x2x8xf32>
    %26 = stablehlo.reshape %25 : (tensor<1x2x8xf32>) -> tensor<2x8xf32>
    %27 = stablehlo.reshape %22 : (tensor<8xf32>) -> tensor<1x8xf32>
    %28 = stablehlo.concatenate %26, %27, dim = 0 : (tensor<2x8xf32>, tensor<1x8xf32>) -> tensor<3x8xf32>
    %29 = stablehlo.slice %arg12 [0:1, 0:2, 0:8] : (tensor<2x2x8xf32>) -> tensor<1x2x8xf32>
    %30 = stablehlo.reshape %29 : (tensor<1x2x8xf32>) -> tensor<2x8xf32>
    %31 = stablehlo.reshape %18 : (tensor<8xf32>) -> tensor<1x8xf32>
    %32 = stablehlo.concatenate %30, %31, dim = 0 : (tensor<2x8xf32>, tensor<1x8xf32>) -> tensor<3x8xf32>
    %33 = stablehlo.slice %24 [0:4] : (tensor<8xf32>) -> tensor<4xf32>
    %34 = stablehlo.slice %28 [0:3, 0:4] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %35 = stablehlo.dot_general %34, %33, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<4xf32>) -> tensor<3xf32>
    %cst_4 = stablehlo.constant dense<2.000000e+00> : tensor<f32>
    %36 = stablehlo.broadcast_in_dim %cst_4, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %37 = stablehlo.divide %35, %36 : tensor<3xf32>
    %cst_5 = stablehlo.constant dense<-inf> : tensor<f32>
    %38 = stablehlo.reduce(%37 init: %cst_5) applies stablehlo.maximum across dimensions = [0] : (tensor<3xf32>, tensor<f32>) -> tensor<f32>
    %39 = stablehlo.broadcast_in_dim %38, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %40 = stablehlo.subtract %37, %39 : tensor<3xf32>
    %41 = stablehlo.exponential %40 : tensor<3xf32>
    %42 = stablehlo.slice %41 [0:1] : (tensor<3xf32>) -> tensor<1xf32>
    %43 = stablehlo.reshape %42 : (tensor<1xf32>) -> tensor<f32>
    %cst_6 = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %44 = stablehlo.add %cst_6, %43 : tensor<f32>
    %45 = stablehlo.slice %41 [1:2] : (tensor<3xf32>) -> tensor<1xf32>
    %46 = stablehlo.reshape %45 : (tensor<1xf32>) -> tensor<f32>
    %47 = stablehlo.add %44, %46 : tensor<f32>
    %48 = stablehlo.slice %41 [2:3] : (tensor<3xf32>) -> tensor<1xf32>
    %49 = stablehlo.reshape %48 : (tensor<1xf32>) -> tensor<f32>
    %50 = stablehlo.add %47, %49 : tensor<f32>
    %51 = stablehlo.broadcast_in_dim %50, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %52 = stablehlo.divide %41, %51 : tensor<3xf32>
    %53 = stablehlo.slice %32 [0:3, 0:4] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %54 = stablehlo.dot_general %53, %52, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<3xf32>) -> tensor<4xf32>
    %55 = stablehlo.slice %24 [4:8] : (tensor<8xf32>) -> tensor<4xf32>
    %56 = stablehlo.slice %28 [0:3, 4:8] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %57 = stablehlo.dot_general %56, %55, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<4xf32>) -> tensor<3xf32>
    %cst_7 = stablehlo.constant dense<2.000000e+00> : tensor<f32>
    %58 = stablehlo.broadcast_in_dim %cst_7, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %59 = stablehlo.divide %57, %58 : tensor<3xf32>
    %cst_8 = stablehlo.constant dense<-inf> : tensor<f32>
    %60 = stablehlo.reduce(%59 init: %cst_8) applies stablehlo.maximum across dimensions = [0] : (tensor<3xf32>, tensor<f32>) -> tensor<f32>
    %61 = stablehlo.broadcast_in_dim %60, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %62 = stablehlo.subtract %59, %61 : tensor<3xf32>
    %63 = stablehlo.exponential %62 : tensor<3xf32>
    %64 = stablehlo.slice %63 [0:1] : (tensor<3xf32>) -> tensor<1xf32>
    %65 = stablehlo.reshape %64 : (tensor<1xf32>) -> tensor<f32>
    %cst_9 = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %66 = stablehlo.add %cst_9, %65 : tensor<f32>
    %67 = stablehlo.slice %63 [1:2] : (tensor<3xf32>) -> tensor<1xf32>
    %68 = stablehlo.reshape %67 : (tensor<1xf32>) -> tensor<f32>
    %69 = stablehlo.add %66, %68 : tensor<f32>
    %70 = stablehlo.slice %63 [2:3] : (tensor<3xf32>) -> tensor<1xf32>
    %71 = stablehlo.reshape %70 : (tensor<1xf32>) -> tensor<f32>
    %72 = stablehlo.add %69, %71 : tensor<f32>
    %73 = stablehlo.broadcast_in_dim %72, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %74 = stablehlo.divide %63, %73 : tensor<3xf32>
    %75 = stablehlo.slice %32 [0:3, 4:8] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %76 = stablehlo.dot_general %75, %74, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<3xf32>) -> tensor<4xf32>
    %77 = stablehlo.concatenate %54, %76, dim = 0 : (tensor<4xf32>, tensor<4xf32>) -> tensor<8xf32>
    %78 = stablehlo.slice %arg8 [0:1, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %79 = stablehlo.reshape %78 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %80 = stablehlo.dot_general %79, %77, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %81 = stablehlo.add %arg0, %80 : tensor<8xf32>
    %82 = stablehlo.slice %arg2 [0:1, 0:8] : (tensor<2x8xf32>) -> tensor<1x8xf32>
    %83 = stablehlo.reshape %82 : (tensor<1x8xf32>) -> tensor<8xf32>
    %84 = stablehlo.dot_general %81, %81, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8xf32>, tensor<8xf32>) -> tensor<f32>
    %cst_10 = stablehlo.constant dense<8.000000e+00> : tensor<f32>
    %85 = stablehlo.divide %84, %cst_10 : tensor<f32>
    %cst_11 = stablehlo.constant dense<1.000000e-05> : tensor<f32>
    %86 = stablehlo.add %85, %cst_11 : tensor<f32>
    %87 = stablehlo.sqrt %86 : tensor<f32>
    %cst_12 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %88 = stablehlo.divide %cst_12, %87 : tensor<f32>
    %89 = stablehlo.multiply %83, %81 : tensor<8xf32>
    %90 = stablehlo.broadcast_in_dim %88, dims = [] : (tensor<f32>) -> tensor<8xf32>
    %91 = stablehlo.multiply %89, %90 : tensor<8xf32>
    %92 = stablehlo.slice %arg4 [0:1, 0:16, 0:8] : (tensor<2x16x8xf32>) -> tensor<1x16x8xf32>
    %93 = stablehlo.reshape %92 : (tensor<1x16x8xf32>) -> tensor<16x8xf32>
    %94 = stablehlo.dot_general %93, %91, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<16x8xf32>, tensor<8xf32>) -> tensor<16xf32>
    %95 = stablehlo.slice %arg6 [0:1, 0:16, 0:8] : (tensor<2x16x8xf32>) -> tensor<1x16x8xf32>
    %96 = stablehlo.reshape %95 : (tensor<1x16x8xf32>) -> tensor<16x8xf32>
    %97 = stablehlo.dot_general %96, %91, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<16x8xf32>, tensor<8xf32>) -> tensor<16xf32>
    %98 = stablehlo.negate %94 : tensor<16xf32>
    %99 = stablehlo.exponential %98 : tensor<16xf32>
    %cst_13 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %100 = stablehlo.broadcast_in_dim %cst_13, dims = [] : (tensor<f32>) -> tensor<16xf32>
    %101 = stablehlo.add %100, %99 : tensor<16xf32>
    %cst_14 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %102 = stablehlo.broadcast_in_dim %cst_14, dims = [] : (tensor<f32>) -> tensor<16xf32>
    %103 = stablehlo.divide %102, %101 : tensor<16xf32>
    %104 = stablehlo.multiply %94, %103 : tensor<16xf32>
    %105 = stablehlo.multiply %104, %97 : tensor<16xf32>
    %106 = stablehlo.slice %arg5 [0:1, 0:8, 0:16] : (tensor<2x8x16xf32>) -> tensor<1x8x16xf32>
    %107 = stablehlo.reshape %106 : (tensor<1x8x16xf32>) -> tensor<8x16xf32>
    %108 = stablehlo.dot_general %107, %105, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x16xf32>, tensor<16xf32>) -> tensor<8xf32>
    %109 = stablehlo.add %81, %108 : tensor<8xf32>
    %110 = stablehlo.slice %arg1 [1:2, 0:8] : (tensor<2x8xf32>) -> tensor<1x8xf32>
    %111 = stablehlo.reshape %110 : (tensor<1x8xf32>) -> tensor<8xf32>
    %112 = stablehlo.dot_general %109, %109, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8xf32>, tensor<8xf32>) -> tensor<f32>
    %cst_15 = stablehlo.constant dense<8.000000e+00> : tensor<f32>
    %113 = stablehlo.divide %112, %cst_15 : tensor<f32>
    %cst_16 = stablehlo.constant dense<1.000000e-05> : tensor<f32>
    %114 = stablehlo.add %113, %cst_16 : tensor<f32>
    %115 = stablehlo.sqrt %114 : tensor<f32>
    %cst_17 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %116 = stablehlo.divide %cst_17, %115 : tensor<f32>
    %117 = stablehlo.multiply %111, %109 : tensor<8xf32>
    %118 = stablehlo.broadcast_in_dim %116, dims = [] : (tensor<f32>) -> tensor<8xf32>
    %119 = stablehlo.multiply %117, %118 : tensor<8xf32>
    %120 = stablehlo.slice %arg9 [1:2, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %121 = stablehlo.reshape %120 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %122 = stablehlo.dot_general %121, %119, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %123 = stablehlo.slice %arg7 [1:2, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %124 = stablehlo.reshape %123 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %125 = stablehlo.dot_general %124, %119, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %126 = stablehlo.slice %arg10 [1:2, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %127 = stablehlo.reshape %126 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %128 = stablehlo.dot_general %127, %119, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %129 = stablehlo.reshape %122 : (tensor<8xf32>) -> tensor<4x2xf32>
    %130 = stablehlo.reshape %125 : (tensor<8xf32>) -> tensor<4x2xf32>
    %cst_18 = stablehlo.constant dense<[[[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]], [[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]]]> : tensor<4x2x2xf32>
    %131 = stablehlo.dot_general %cst_18, %130, batching_dims = [0] x [0], contracting_dims = [2] x [1], precision = [DEFAULT, DEFAULT] : (tensor<4x2x2xf32>, tensor<4x2xf32>) -> tensor<4x2xf32>
    %132 = stablehlo.reshape %131 : (tensor<4x2xf32>) -> tensor<8xf32>
    %cst_19 = stablehlo.constant dense<[[[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]], [[-4.161468e-01, -9.092974e-01], [9.092974e-01, -4.161468e-01]], [[9.998000e-01, -1.999867e-02], [1.999867e-02, 9.998000e-01]]]> : tensor<4x2x2xf32>
    %133 = stablehlo.dot_general %cst_19, %129, batching_dims = [0] x [0], contracting_dims = [2] x [1], precision = [DEFAULT, DEFAULT] : (tensor<4x2x2xf32>, tensor<4x2xf32>) -> tensor<4x2xf32>
    %134 = stablehlo.reshape %133 : (tensor<4x2xf32>) -> tensor<8xf32>
    %135 = stablehlo.slice %arg11 [1:2, 0:2, 0:8] : (tensor<2x2x8xf32>) -> tensor<1x2x8xf32>
    %136 = stablehlo.reshape %135 : (tensor<1x2x8xf32>) -> tensor<2x8xf32>
    %137 = stablehlo.reshape %132 : (tensor<8xf32>) -> tensor<1x8xf32>
    %138 = stablehlo.concatenate %136, %137, dim = 0 : (tensor<2x8xf32>, tensor<1x8xf32>) -> tensor<3x8xf32>
    %139 = stablehlo.slice %arg12 [1:2, 0:2, 0:8] : (tensor<2x2x8xf32>) -> tensor<1x2x8xf32>
    %140 = stablehlo.reshape %139 : (tensor<1x2x8xf32>) -> tensor<2x8xf32>
    %141 = stablehlo.reshape %128 : (tensor<8xf32>) -> tensor<1x8xf32>
    %142 = stablehlo.concatenate %140, %141, dim = 0 : (tensor<2x8xf32>, tensor<1x8xf32>) -> tensor<3x8xf32>
    %143 = stablehlo.slice %134 [0:4] : (tensor<8xf32>) -> tensor<4xf32>
    %144 = stablehlo.slice %138 [0:3, 0:4] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %145 = stablehlo.dot_general %144, %143, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<4xf32>) -> tensor<3xf32>
    %cst_20 = stablehlo.constant dense<2.000000e+00> : tensor<f32>
    %146 = stablehlo.broadcast_in_dim %cst_20, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %147 = stablehlo.divide %145, %146 : tensor<3xf32>
    %cst_21 = stablehlo.constant dense<-inf> : tensor<f32>
    %148 = stablehlo.reduce(%147 init: %cst_21) applies stablehlo.maximum across dimensions = [0] : (tensor<3xf32>, tensor<f32>) -> tensor<f32>
    %149 = stablehlo.broadcast_in_dim %148, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %150 = stablehlo.subtract %147, %149 : tensor<3xf32>
    %151 = stablehlo.exponential %150 : tensor<3xf32>
    %152 = stablehlo.slice %151 [0:1] : (tensor<3xf32>) -> tensor<1xf32>
    %153 = stablehlo.reshape %152 : (tensor<1xf32>) -> tensor<f32>
    %cst_22 = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %154 = stablehlo.add %cst_22, %153 : tensor<f32>
    %155 = stablehlo.slice %151 [1:2] : (tensor<3xf32>) -> tensor<1xf32>
    %156 = stablehlo.reshape %155 : (tensor<1xf32>) -> tensor<f32>
    %157 = stablehlo.add %154, %156 : tensor<f32>
    %158 = stablehlo.slice %151 [2:3] : (tensor<3xf32>) -> tensor<1xf32>
    %159 = stablehlo.reshape %158 : (tensor<1xf32>) -> tensor<f32>
    %160 = stablehlo.add %157, %159 : tensor<f32>
    %161 = stablehlo.broadcast_in_dim %160, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %162 = stablehlo.divide %151, %161 : tensor<3xf32>
    %163 = stablehlo.slice %142 [0:3, 0:4] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %164 = stablehlo.dot_general %163, %162, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<3xf32>) -> tensor<4xf32>
    %165 = stablehlo.slice %134 [4:8] : (tensor<8xf32>) -> tensor<4xf32>
    %166 = stablehlo.slice %138 [0:3, 4:8] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %167 = stablehlo.dot_general %166, %165, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<4xf32>) -> tensor<3xf32>
    %cst_23 = stablehlo.constant dense<2.000000e+00> : tensor<f32>
    %168 = stablehlo.broadcast_in_dim %cst_23, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %169 = stablehlo.divide %167, %168 : tensor<3xf32>
    %cst_24 = stablehlo.constant dense<-inf> : tensor<f32>
    %170 = stablehlo.reduce(%169 init: %cst_24) applies stablehlo.maximum across dimensions = [0] : (tensor<3xf32>, tensor<f32>) -> tensor<f32>
    %171 = stablehlo.broadcast_in_dim %170, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %172 = stablehlo.subtract %169, %171 : tensor<3xf32>
    %173 = stablehlo.exponential %172 : tensor<3xf32>
    %174 = stablehlo.slice %173 [0:1] : (tensor<3xf32>) -> tensor<1xf32>
    %175 = stablehlo.reshape %174 : (tensor<1xf32>) -> tensor<f32>
    %cst_25 = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %176 = stablehlo.add %cst_25, %175 : tensor<f32>
    %177 = stablehlo.slice %173 [1:2] : (tensor<3xf32>) -> tensor<1xf32>
    %178 = stablehlo.reshape %177 : (tensor<1xf32>) -> tensor<f32>
    %179 = stablehlo.add %176, %178 : tensor<f32>
    %180 = stablehlo.slice %173 [2:3] : (tensor<3xf32>) -> tensor<1xf32>
    %181 = stablehlo.reshape %180 : (tensor<1xf32>) -> tensor<f32>
    %182 = stablehlo.add %179, %181 : tensor<f32>
    %183 = stablehlo.broadcast_in_dim %182, dims = [] : (tensor<f32>) -> tensor<3xf32>
    %184 = stablehlo.divide %173, %183 : tensor<3xf32>
    %185 = stablehlo.slice %142 [0:3, 4:8] : (tensor<3x8xf32>) -> tensor<3x4xf32>
    %186 = stablehlo.dot_general %185, %184, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<3x4xf32>, tensor<3xf32>) -> tensor<4xf32>
    %187 = stablehlo.concatenate %164, %186, dim = 0 : (tensor<4xf32>, tensor<4xf32>) -> tensor<8xf32>
    %188 = stablehlo.slice %arg8 [1:2, 0:8, 0:8] : (tensor<2x8x8xf32>) -> tensor<1x8x8xf32>
    %189 = stablehlo.reshape %188 : (tensor<1x8x8xf32>) -> tensor<8x8xf32>
    %190 = stablehlo.dot_general %189, %187, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %191 = stablehlo.add %109, %190 : tensor<8xf32>
    %192 = stablehlo.slice %arg2 [1:2, 0:8] : (tensor<2x8xf32>) -> tensor<1x8xf32>
    %193 = stablehlo.reshape %192 : (tensor<1x8xf32>) -> tensor<8xf32>
    %194 = stablehlo.dot_general %191, %191, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8xf32>, tensor<8xf32>) -> tensor<f32>
    %cst_26 = stablehlo.constant dense<8.000000e+00> : tensor<f32>
    %195 = stablehlo.divide %194, %cst_26 : tensor<f32>
    %cst_27 = stablehlo.constant dense<1.000000e-05> : tensor<f32>
    %196 = stablehlo.add %195, %cst_27 : tensor<f32>
    %197 = stablehlo.sqrt %196 : tensor<f32>
    %cst_28 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %198 = stablehlo.divide %cst_28, %197 : tensor<f32>
    %199 = stablehlo.multiply %193, %191 : tensor<8xf32>
    %200 = stablehlo.broadcast_in_dim %198, dims = [] : (tensor<f32>) -> tensor<8xf32>
    %201 = stablehlo.multiply %199, %200 : tensor<8xf32>
    %202 = stablehlo.slice %arg4 [1:2, 0:16, 0:8] : (tensor<2x16x8xf32>) -> tensor<1x16x8xf32>
    %203 = stablehlo.reshape %202 : (tensor<1x16x8xf32>) -> tensor<16x8xf32>
    %204 = stablehlo.dot_general %203, %201, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<16x8xf32>, tensor<8xf32>) -> tensor<16xf32>
    %205 = stablehlo.slice %arg6 [1:2, 0:16, 0:8] : (tensor<2x16x8xf32>) -> tensor<1x16x8xf32>
    %206 = stablehlo.reshape %205 : (tensor<1x16x8xf32>) -> tensor<16x8xf32>
    %207 = stablehlo.dot_general %206, %201, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<16x8xf32>, tensor<8xf32>) -> tensor<16xf32>
    %208 = stablehlo.negate %204 : tensor<16xf32>
    %209 = stablehlo.exponential %208 : tensor<16xf32>
    %cst_29 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %210 = stablehlo.broadcast_in_dim %cst_29, dims = [] : (tensor<f32>) -> tensor<16xf32>
    %211 = stablehlo.add %210, %209 : tensor<16xf32>
    %cst_30 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %212 = stablehlo.broadcast_in_dim %cst_30, dims = [] : (tensor<f32>) -> tensor<16xf32>
    %213 = stablehlo.divide %212, %211 : tensor<16xf32>
    %214 = stablehlo.multiply %204, %213 : tensor<16xf32>
    %215 = stablehlo.multiply %214, %207 : tensor<16xf32>
    %216 = stablehlo.slice %arg5 [1:2, 0:8, 0:16] : (tensor<2x8x16xf32>) -> tensor<1x8x16xf32>
    %217 = stablehlo.reshape %216 : (tensor<1x8x16xf32>) -> tensor<8x16xf32>
    %218 = stablehlo.dot_general %217, %215, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8x16xf32>, tensor<16xf32>) -> tensor<8xf32>
    %219 = stablehlo.add %191, %218 : tensor<8xf32>
    %220 = stablehlo.dot_general %219, %219, contracting_dims = [0] x [0], precision = [DEFAULT, DEFAULT] : (tensor<8xf32>, tensor<8xf32>) -> tensor<f32>
    %cst_31 = stablehlo.constant dense<8.000000e+00> : tensor<f32>
    %221 = stablehlo.divide %220, %cst_31 : tensor<f32>
    %cst_32 = stablehlo.constant dense<1.000000e-05> : tensor<f32>
    %222 = stablehlo.add %221, %cst_32 : tensor<f32>
    %223 = stablehlo.sqrt %222 : tensor<f32>
    %cst_33 = stablehlo.constant dense<1.000000e+00> : tensor<f32>
    %224 = stablehlo.divide %cst_33, %223 : tensor<f32>
    %225 = stablehlo.multiply %arg3, %219 : tensor<8xf32>
    %226 = stablehlo.broadcast_in_dim %224, dims = [] : (tensor<f32>) -> tensor<8xf32>
    %227 = stablehlo.multiply %225, %226 : tensor<8xf32>
    return %227 : tensor<8xf32>
  }
}
