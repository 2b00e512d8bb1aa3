"""Regenerates tests/golden from the reference checkout (run in the build container only).

    python tests/golden/make_golden.py [path of the reference checkout]

1. fixtures/*.param are the reference's own operator fixtures for the hot path
   (test/Numerical/fixtures), copied as data; fixtures/*.bin are produced by RUNNING
   the reference's generators (generate_bins.py, generate_int8_bins.py).
2. loader_dumps/*.txt is the output of oracle/_ref/ref_dump -- the reference's own
   lib/Graph loader compiled from its sources -- on every fixture, on malformed
   variants, and on the synthetic benchmark models written by the package's zoo.
Nothing at test time reads the reference checkout; only these files travel.
"""
import importlib.util
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("NCNN_COMPILER_REFERENCE") or
                                             os.path.join(os.path.dirname(ROOT), "reference"))
FIX = os.path.join(REF, "test", "Numerical", "fixtures")

F32_CASES = ["convolution", "convolution_no_bias", "convolution_dilated", "convolution_asymmetric",
             "convolution_asymmetric_stride", "convolution_same_upper", "convolution_same_lower",
             "convolution_fp16_storage", "convolution_depthwise", "convolution_depthwise_fp16_storage",
             "convolution_depthwise_7x7", "convolution_depthwise_asymmetric",
             "convolution_depthwise_same_upper", "convolution_depthwise_same_lower", "inner_product",
             "inner_product_dynamic_m", "inner_product_fused_relu", "batch_norm", "gemm", "deconvolution",
             "deconvolution_no_bias", "deconvolution_tiny_head"]
INT8_CASES = ["convolution_int8_term1", "convolution_int8_term2", "convolution_int8_term101",
              "convolution_int8_term102", "depthwise_int8_term1", "depthwise_int8_term2",
              "depthwise_int8_term101", "depthwise_int8_term102", "inner_product_int8_term1",
              "inner_product_int8_term2", "int8_complete_chain", "gemm_int8_term2"]
NO_WEIGHTS = ["pooling", "pooling_tail", "pooling_average", "pooling_asymmetric", "pooling_global_average",
              "pooling_global_average_ignored_params", "pooling_global_max", "pooling_global_max_ignored_params",
              "pooling_same_upper", "pooling_same_lower", "eltwise_weighted", "binary_add", "binary_mul_scalar",
              "relu", "relu_leaky", "split", "reshape", "squeeze", "permute", "expand_dims", "gelu",
              "sigmoid", "hard_sigmoid", "hard_swish", "dropout", "softmax", "softmax_channel", "softmax_height",
              "softmax_width", "softmax_negative_channel", "softmax_negative_height", "softmax_negative_width",
              "concat", "concat_height", "concat_width", "concat_negative_channel", "concat_negative_height",
              "concat_negative_width", "split_three", "binary_mul_channel", "binary_mul_reverse_broadcast",
              "unary_square", "slice", "shuffle_channel", "shuffle_channel_reverse", "padding", "padding_four_sides",
              "padding_identity", "interp", "interp_asymmetric", "interp_eightfold", "interp_explicit_target",
              "interp_identity", "reduction_mean", "reduction_mean_keepdims_coeff"]


def main():
    out_fix = os.path.join(HERE, "fixtures")
    out_dump = os.path.join(HERE, "loader_dumps")
    for d in (out_fix, out_dump):
        shutil.rmtree(d, ignore_errors=True)
        os.makedirs(d)
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "ref", f"REFERENCE={REF}"])
    ref_dump = os.path.join(ROOT, "oracle", "_ref", "ref_dump")
    for case in F32_CASES + INT8_CASES + NO_WEIGHTS:
        shutil.copy(os.path.join(FIX, case + ".param"), os.path.join(out_fix, case + ".param"))
    for case in F32_CASES:
        subprocess.check_call([sys.executable, os.path.join(FIX, "generate_bins.py"),
                               os.path.join(out_fix, case + ".bin"), case])
    for case in INT8_CASES:
        subprocess.check_call([sys.executable, os.path.join(FIX, "generate_int8_bins.py"),
                               os.path.join(out_fix, case + ".bin"), case])
    for case in NO_WEIGHTS:
        open(os.path.join(out_fix, case + ".bin"), "wb").close()

    def dump(name, param, bin_path):
        args = [ref_dump, param] + ([bin_path] if bin_path else [])
        text = subprocess.run(args, capture_output=True, text=True).stdout
        with open(os.path.join(out_dump, name + ".txt"), "w") as f:
            f.write(text)

    for case in F32_CASES + INT8_CASES + NO_WEIGHTS:
        dump(case, os.path.join(out_fix, case + ".param"), os.path.join(out_fix, case + ".bin"))
    # every other fixture of the reference, parsed without weights (grammar coverage)
    for name in sorted(os.listdir(FIX)):
        if name.endswith(".param") and name[:-6] not in F32_CASES + INT8_CASES + NO_WEIGHTS:
            shutil.copy(os.path.join(FIX, name), os.path.join(out_fix, name))
            dump(name[:-6] + ".nobin", os.path.join(out_fix, name), None)

    # malformed inputs: what the reference's loader answers
    tmp = os.path.join(out_fix, "_malformed")
    os.makedirs(tmp)
    conv_param = open(os.path.join(out_fix, "convolution.param")).read()
    conv_bin = open(os.path.join(out_fix, "convolution.bin"), "rb").read()
    variants = {
        "bad_magic": (conv_param.replace("7767517", "7767518"), conv_bin),
        "truncated_bin": (conv_param, conv_bin[:-4]),
        "oversized_bin": (conv_param, conv_bin + b"\0\0\0\0"),
        "missing_layer": (conv_param.replace("2 2", "3 2", 1), conv_bin),
        "too_many_blobs": (conv_param.replace("2 2", "2 1", 1), conv_bin),
        "unresolved_bottom": (conv_param.replace("1 1 data output", "1 1 nodata output"), conv_bin),
        "bad_param_value": (conv_param.replace("0=2 1=3", "0=2 1=x3"), conv_bin),
        "missing_equals": (conv_param.replace("0=2 1=3", "0=2 13"), conv_bin),
        "array_length_mismatch": (conv_param.replace(" 6=18", " 6=18 -23310=3,1.0,2.0"), conv_bin),
        "float_for_int": (conv_param.replace("0=2 1=3", "0=2.0 1=3"), conv_bin),
        "bad_weight_flag": (conv_param, b"\x01\x02\x03\x04" + conv_bin[4:]),
        "empty": ("", conv_bin),
        "short_layer_line": (conv_param.replace("Convolution convolution 1 1 data output", "Convolution convolution 1"), conv_bin),
    }
    for name, (ptxt, bdata) in variants.items():
        p = os.path.join(tmp, name + ".param")
        b = os.path.join(tmp, name + ".bin")
        open(p, "w").write(ptxt)
        open(b, "wb").write(bdata)
        dump("_malformed_" + name, p, b)

    # synthetic benchmark models (small spatial size keeps the files out of the repo;
    # the dump pins layer structure, parameter typing and weight hashes)
    spec = importlib.util.spec_from_file_location("zoo", os.path.join(ROOT, "ncnn-compiler_b200", "zoo.py"))
    zoo = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(zoo)
    ztmp = os.path.join("/tmp", "golden_zoo")
    os.makedirs(ztmp, exist_ok=True)
    for name, fn, kw in [("zoo_single_conv", zoo.single_conv, {}), ("zoo_resnet18", zoo.resnet18, {}),
                         ("zoo_resnet18_int8", zoo.resnet18, {"int8": True}),
                         ("zoo_mobilenet_v2", zoo.mobilenet_v2, {}),
                         ("zoo_inner_product", lambda p: zoo.inner_product(p, 512, 1024), {}),
                         ("zoo_inner_product_int8", lambda p: zoo.inner_product(p, 512, 1024, int8=True), {})]:
        p, b = fn(os.path.join(ztmp, name), **kw)
        dump(name, p, b)


if __name__ == "__main__":
    main()
