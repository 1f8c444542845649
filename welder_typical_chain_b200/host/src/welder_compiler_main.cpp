// welder-compiler: CLI over welderCompilerMain, for the process_chain backend mode.
#include "../../../include/welder_compile_capi.h"

int main(int argc, char **argv) { return welderCompilerMain(argc, argv); }
