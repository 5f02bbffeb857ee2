"""gen_ir stand-in (pycuke1/asg2ir.py:192): cuke lowers the graph to a loop IR here; the prebuilt kernels
need no IR, so the graph is returned unchanged and recognition happens in codegen.gpu.print_cuda."""


def gen_ir(node):
    node.eval = node
    return node
