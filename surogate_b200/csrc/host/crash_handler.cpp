// Fatal-signal handler that prints the signal, the rank and a native stack trace to stderr before re-raising with the
// default action, so a crash inside a worker leaves a trace in the job log.
// Reference counterpart: csrc/src/utilities/crash_handler.h:26.
#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>

#include "host_api.h"

namespace sg {

static char g_tag[128] = "surogate_b200";

static void on_fatal(int sig) {
    char line[256];
    int n = snprintf(line, sizeof line, "\n[%s] fatal signal %d (%s); native stack:\n", g_tag, sig, strsignal(sig));
    if (n > 0) (void)!write(STDERR_FILENO, line, static_cast<size_t>(n));
    void* frames[64];
    int depth = backtrace(frames, 64);
    backtrace_symbols_fd(frames, depth, STDERR_FILENO);
    signal(sig, SIG_DFL);
    raise(sig);
}

void install_crash_handler(const std::string& tag) {
    strncpy(g_tag, tag.c_str(), sizeof(g_tag) - 1);
    void* warm[4];
    backtrace(warm, 4);  // loads libgcc now: not safe to do for the first time inside a handler
    struct sigaction sa;
    memset(&sa, 0, sizeof sa);
    sa.sa_handler = on_fatal;
    sigemptyset(&sa.sa_mask);
    sa.sa_flags = SA_RESETHAND | SA_NODEFER;
    for (int s : {SIGSEGV, SIGBUS, SIGFPE, SIGILL, SIGABRT}) sigaction(s, &sa, nullptr);
}

}  // namespace sg
